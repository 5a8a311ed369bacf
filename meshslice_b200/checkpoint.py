"""Checkpoints: one file per mesh coordinate plus a ``meta.json``, an offline re-sharder and an
importer for per-device blocks exported from the JAX reference.

The reference has no save/load at all; what it fixes is the parameter layout per mesh
coordinate, which this format keeps (ShardedLayers.py:33-36, 93-100, 152-153):

* a linear weight is one 2-D array sharded P(row, col): coordinate (r, c) holds the contiguous
  block ``W[r*d0/R:(r+1)*d0/R, c*d1/C:(c+1)*d1/C]``; the global orientation is [out, in] for
  dataflow 'ls' and [in, out] otherwise;
* QKV columns are ordered per head [q | k | v];
* LayerNorm / embedding parameters are P(None, col): coordinate (r, c) holds columns
  ``[c*n/C:(c+1)*n/C]`` and every row index holds the same values.

Layout on disk: ``<dir>/step_<N>/shard_r<r>_c<c>.pt`` = {name: local block} plus, when an
optimizer is saved, ``optim/master/<name>``, ``optim/m/<name>``, ``optim/v/<name>`` (fp32, same
block as the parameter, so the optimizer state re-shards with the parameters) and
``optim/step``; ``<dir>/step_<N>/meta.json`` (mesh, per-parameter global shape / kind / dataflow /
dtype, step, whether optimizer state is present, caller's ``extra`` such as the data position).
meta.json is written last, through a temporary file and an atomic rename: a step directory
without it is an interrupted save.

Loading parameters without optimizer state (an older checkpoint, imported weights) rebuilds the
optimizer's fp32 master copies from the loaded parameters and clears the moments.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

import torch

from .parallel.mesh import Mesh, ShardedTensor


def _step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"step_{step}")


def _global_shape(local_shape, kind: str, R: int, C: int):
    if kind == "sharded":
        return [local_shape[0] * R, local_shape[1] * C]
    s = list(local_shape)
    s[-1] *= C
    return s


_OPT_KEYS = ("master", "m", "v")


def save_checkpoint(root: str, step: int, model, optimizer=None, extra: Optional[dict] = None, rank0: bool = True,
                    barrier=None):
    """Every process writes the coordinates it holds; the process with ``rank0`` writes meta.json
    after ``barrier()`` (when given: a callable that returns once every process has written its
    shard files, e.g. ``torch.distributed.barrier``)."""
    mesh: Mesh = model.mesh
    d = _step_dir(root, step)
    os.makedirs(d, exist_ok=True)
    params = model.parameters()
    named = optimizer.named_state(params) if optimizer is not None else None
    for (r, c) in mesh.coords():
        blob = {name: p.shards[(r, c)].detach().cpu() for name, p, _, _ in params}
        if optimizer is not None:
            blob["optim/step"] = torch.tensor(optimizer.step_count)
            for name, per in named.items():
                for k, view in zip(_OPT_KEYS, per[(r, c)]):
                    blob[f"optim/{k}/{name}"] = view.detach().cpu().clone()
        tmp = os.path.join(d, f".shard_r{r}_c{c}.pt.tmp")
        torch.save(blob, tmp)
        os.replace(tmp, os.path.join(d, f"shard_r{r}_c{c}.pt"))
    if barrier is not None:
        barrier()
    if rank0:
        meta = {"format": "meshslice_b200.ckpt.v1", "mesh": [mesh.R, mesh.C], "step": step,
                "has_optimizer": optimizer is not None, "extra": extra or {}, "params": {}}
        dataflows = {}
        for i, b in enumerate(getattr(model, "blocks", [])):
            for j, l in enumerate(b.layers()):
                if hasattr(l, "dataflow"):
                    dataflows[f"block{i}.{type(l).__name__}{j}.weight"] = l.dataflow
        if hasattr(model, "head"):
            dataflows["head.weight"] = model.head.dataflow
        for name, p, _, kind in params:
            local = next(iter(p.shards.values()))
            meta["params"][name] = {"kind": kind, "dtype": str(local.dtype).replace("torch.", ""),
                                    "global_shape": _global_shape(local.shape, kind, mesh.R, mesh.C),
                                    "dataflow": dataflows.get(name),
                                    "orientation": "[out,in]" if dataflows.get(name) == "ls" else "[in,out]"
                                    if name in dataflows else None}
        _write_json_atomic(os.path.join(d, "meta.json"), meta)
    return d


def _write_json_atomic(path: str, obj):
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(obj, f, indent=1)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def load_checkpoint(root: str, step: int, model, optimizer=None) -> dict:
    """Loads the coordinates this process holds.  Raises if the mesh shape or a shard shape
    does not match (re-shard offline with ``reshard_checkpoint`` first)."""
    mesh: Mesh = model.mesh
    d = _step_dir(root, step)
    meta = json.load(open(os.path.join(d, "meta.json")))
    if meta["mesh"] != [mesh.R, mesh.C]:
        raise ValueError(f"checkpoint mesh {meta['mesh']} != model mesh {[mesh.R, mesh.C]}; re-shard it first")
    params = model.parameters()
    with_opt = optimizer is not None and bool(meta.get("has_optimizer"))
    named = optimizer.named_state(params) if with_opt else None
    for (r, c) in mesh.coords():
        path = os.path.join(d, f"shard_r{r}_c{c}.pt")
        if not os.path.exists(path):
            raise FileNotFoundError(f"missing shard file {path}")
        try:
            blob = torch.load(path, map_location="cpu")
        except Exception as e:
            raise RuntimeError(f"corrupted shard file {path}: {e}") from e
        for name, p, _, _ in params:
            if name not in blob:
                raise KeyError(f"{path} has no parameter {name}")
            t = p.shards[(r, c)]
            if tuple(blob[name].shape) != tuple(t.shape):
                raise ValueError(f"{name}: shard shape {tuple(blob[name].shape)} != {tuple(t.shape)}")
            t.copy_(blob[name].to(t.dtype))
        if with_opt:
            optimizer.step_count = int(blob["optim/step"])
            for name, per in named.items():
                for k, view in zip(_OPT_KEYS, per[(r, c)]):
                    key = f"optim/{k}/{name}"
                    if key not in blob:
                        raise KeyError(f"{path} has no optimizer state {key}")
                    view.copy_(blob[key].to(view.dtype))
    if optimizer is not None and not with_opt:
        # no optimizer state on disk: without this the first step would write the stale fp32
        # master copies (the construction-time weights) over the parameters just loaded
        optimizer.resync_from_params(step=int(meta.get("step", 0)))
    return meta


def _assemble(blobs: Dict[Tuple[int, int], dict], name: str, kind: str, R: int, C: int) -> torch.Tensor:
    if kind == "sharded":
        return torch.cat([torch.cat([blobs[(r, c)][name] for c in range(C)], dim=1) for r in range(R)], dim=0)
    return torch.cat([blobs[(0, c)][name] for c in range(C)], dim=-1)


def _split(full: torch.Tensor, kind: str, R: int, C: int, r: int, c: int) -> torch.Tensor:
    if kind == "sharded":
        b0, b1 = full.shape[0] // R, full.shape[1] // C
        return full[r * b0:(r + 1) * b0, c * b1:(c + 1) * b1].clone()
    b = full.shape[-1] // C
    return full[..., c * b:(c + 1) * b].clone()


def reshard_checkpoint(root: str, step: int, new_mesh: Tuple[int, int], out_root: str) -> str:
    """Offline R x C -> R' x C' conversion of the parameters and, when present, of the optimizer
    state (fp32 master copies and both moments are stored per parameter with the parameter's own
    sharding, so they are cut the same way)."""
    d = _step_dir(root, step)
    meta = json.load(open(os.path.join(d, "meta.json")))
    R, C = meta["mesh"]
    R2, C2 = new_mesh
    blobs = {(r, c): torch.load(os.path.join(d, f"shard_r{r}_c{c}.pt"), map_location="cpu")
             for r in range(R) for c in range(C)}
    out = _step_dir(out_root, step)
    os.makedirs(out, exist_ok=True)
    kinds = {n: info["kind"] for n, info in meta["params"].items()}
    has_opt = bool(meta.get("has_optimizer"))
    if has_opt:
        for n, info in meta["params"].items():
            for k in _OPT_KEYS:
                kinds[f"optim/{k}/{n}"] = info["kind"]
    fulls = {n: _assemble(blobs, n, kind, R, C) for n, kind in kinds.items()}
    for n, f in fulls.items():
        k = kinds[n]
        if (k == "sharded" and (f.shape[0] % R2 or f.shape[1] % C2)) or (k != "sharded" and f.shape[-1] % C2):
            raise ValueError(f"{n} with global shape {tuple(f.shape)} does not divide over mesh {new_mesh}")
    for r in range(R2):
        for c in range(C2):
            blob = {n: _split(f, kinds[n], R2, C2, r, c) for n, f in fulls.items()}
            if has_opt:
                blob["optim/step"] = blobs[(0, 0)]["optim/step"].clone()
            torch.save(blob, os.path.join(out, f"shard_r{r}_c{c}.pt"))
    _write_json_atomic(os.path.join(out, "meta.json"), dict(meta, mesh=[R2, C2]))
    return out


def import_jax_blocks(block_dir: str, model, name_map: Dict[str, str], optimizer=None) -> List[str]:
    """Loads a pytree exported from the JAX reference as per-device ``.npy`` blocks named
    ``<param>.r<r>.c<c>.npy`` (one file per NamedSharding(mesh, P(row, col)) shard, or
    ``<param>.c<c>.npy`` for P(col) vectors).  ``name_map`` maps this model's parameter names to
    the exported names.  With ``optimizer`` its fp32 master copies are rebuilt from the imported
    parameters.  Returns the parameters that were loaded."""
    import numpy as np
    mesh: Mesh = model.mesh
    loaded = []
    for name, p, _, kind in model.parameters():
        if name not in name_map:
            continue
        for (r, c) in mesh.coords():
            fn = (f"{name_map[name]}.r{r}.c{c}.npy" if kind == "sharded" else f"{name_map[name]}.c{c}.npy")
            path = os.path.join(block_dir, fn)
            if not os.path.exists(path):
                raise FileNotFoundError(path)
            arr = torch.from_numpy(np.load(path).astype("float32"))
            t = p.shards[(r, c)]
            if tuple(arr.shape) != tuple(t.shape):
                raise ValueError(f"{fn}: block shape {tuple(arr.shape)} != {tuple(t.shape)}")
            t.copy_(arr.to(t.dtype))
        loaded.append(name)
    if optimizer is not None:
        optimizer.resync_from_params(step=0)
    return loaded
