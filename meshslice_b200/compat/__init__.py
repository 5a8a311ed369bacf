"""Modules named like the reference's flat scripts, re-exporting this package's equivalents so
that ``from meshslice_b200.compat.TensorParallel import SPMD`` reads like the original import."""
