"""Autotuner: dataflow per linear layer, transposition propagation, mesh shape and slice count
(counterpart of Autotuner.py).

Pipeline as in the reference: (1) pick a dataflow per FeedForward node by keeping the largest of
{input, weight, output} stationary (Autotuner.py:288-302); (2) propagate activation orientation,
inserting Transpose nodes where the inputs of an Add disagree (:304-337); (3) analytically choose
the mesh shape that minimises traffic + latency and, per layer, the slice count that minimises
latency + 2 x pipeline fill (:339-390); (4) refine with the emulated step time from the cost
model around the analytic optimum, or sweep all shapes (:391-483).

What differs from the reference: fabric constants are data (``FabricConstants``, loadable from
the JSON written by ``BenchCollectives2D``) instead of module globals edited by hand; the defects
of the reference are fixed (the 'rs' branch divided by a tuple, :66; ``bestK = K`` used the global
K, :418; ``self.bsetshape`` typo, :440); candidate slice counts are enumerated from divisibility
rather than a lookup table, for any block size; results can be written as JSON
(``--tuned-json``) for the trainer and benchmarks to read.
"""
from __future__ import annotations

import argparse
import copy
import json
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from . import cost_model as CostModel
from .cost_model import DeviceMesh

# TPUv4 fit shipped with the reference (Autotuner.py:17-19), kept for regression tests
TPUV4 = dict(
    latencies={"allgather": 5e-6, "reducescatter": 5e-6, "sendrecv": 5e-5},
    bws={"allgather": (27.472e9, 79.751e9), "reducescatter": (37.506e9, 63.167e9), "sendrecv": (38.801e9, 35.224e9)},
    base_overheads={"allgather": 13e-6, "reducescatter": 26e-6, "sendrecv": 13e-6},
    fabric="ring", shared_port=False, flops_per_chip=242 * 1024 ** 4)

# NVLink 5 / NVSwitch defaults for one 8 x B200 box (measured per-direction peer-copy bandwidth of a
# port: 770 GB/s; refined by BenchCollectives2D --fabric-json)
B200_NVSWITCH = dict(
    latencies={"allgather": 3e-6, "reducescatter": 3e-6, "sendrecv": 3e-6},
    bws={"allgather": (700e9, 700e9), "reducescatter": (600e9, 600e9), "sendrecv": (700e9, 700e9)},
    base_overheads={"allgather": 6e-6, "reducescatter": 8e-6, "sendrecv": 5e-6},
    fabric="switch", shared_port=True, flops_per_chip=1.38e15,
    # rates of the fused GEMM + collective kernel fitted to 2-D GeMM sweeps on 8 and 2 GPUs (bench/fit_fused_model.py)
    fused=dict(launch_overhead=1.82e-05, gather_bw_alone=6.1e+11, gather_bw_overlap=3.08e+11, push_bw=5.88e+11,
               slot_sum_bw=5.81e+11, tile_eff=0.951, slice_overhead=8.51e-06, matmul_peak=1.3806e15))

latencies = TPUV4["latencies"]
bws = TPUV4["bws"]
base_overheads = TPUV4["base_overheads"]


@dataclass
class FabricConstants:
    latencies: Dict[str, float]
    bws: Dict[str, Tuple[float, float]]
    base_overheads: Dict[str, float]
    fabric: str = "ring"
    shared_port: bool = False
    flops_per_chip: float = 242 * 1024 ** 4
    # rates of the fused GEMM + collective kernel (cost_model.FusedKernelConstants as a dict); when present the
    # per-layer emulation models that kernel instead of the collective-then-GEMM pipeline
    fused: Optional[Dict[str, float]] = None

    @classmethod
    def from_dict(cls, d):
        b = {k: tuple(v) if isinstance(v, (list, tuple)) else (v, v) for k, v in d["bws"].items()}
        return cls(d["latencies"], b, d["base_overheads"], d.get("fabric", "ring"), d.get("shared_port", False),
                   d.get("flops_per_chip", 242 * 1024 ** 4), d.get("fused"))

    @classmethod
    def load(cls, path):
        return cls.from_dict(json.load(open(path)))

    def mesh(self, shape, matmul=None) -> DeviceMesh:
        fused = CostModel.FusedKernelConstants(**self.fused) if self.fused else None
        return DeviceMesh(shape, self.flops_per_chip, self.bws, self.latencies, self.base_overheads,
                          fabric=self.fabric, shared_port=self.shared_port, matmul=matmul, fused=fused)


class FFLayerModel:
    """Per-layer traffic / latency / pipeline model over forward, backward-data and
    backward-weight (Autotuner.py:21-169).  B = tokens, I = in features, O = out features."""

    def __init__(self, B, I, O, dataflow=None, transpose=False):
        self.bsize, self.in_dim, self.out_dim = B, I, O
        if dataflow in ("os", "rs", "ls"):
            self.dataflow = dataflow
        elif O > I and B >= I:
            self.dataflow = "os"
        elif I >= O and B >= O:
            self.dataflow = "ls"
        else:                       # the weight is the largest matrix
            self.dataflow = "rs"
        self.transpose = transpose

    # traffic volumes (bytes over the whole mesh) of the two moving matrices and the mesh
    # dimension each travels along: (bytes_a, dim_a, bytes_b, dim_b)
    def _moving(self, mesh: DeviceMesh):
        R, C = mesh.shape
        da, db = (1, 0) if not self.transpose else (0, 1)
        na, nb = mesh.shape[da] - 1, mesh.shape[db] - 1
        if self.dataflow == "os":       # input along columns, weight along rows
            return 2 * self.bsize * self.in_dim * na, da, 2 * self.in_dim * self.out_dim * nb, db
        if self.dataflow == "ls":       # output along columns, weight along rows
            return 2 * self.bsize * self.out_dim * na, da, 2 * self.in_dim * self.out_dim * nb, db
        # 'rs': input along columns, output along rows
        return 2 * self.bsize * self.in_dim * na, da, 2 * self.bsize * self.out_dim * nb, db

    # which collective moves (matrix a, matrix b) in (forward, backward-data, backward-weight)
    def _kinds(self):
        AG, RS = "allgather", "reducescatter"
        if self.dataflow == "os":
            return ((AG, AG), (RS, AG), (AG, RS))
        if self.dataflow == "ls":
            return ((RS, AG), (AG, AG), (AG, RS))
        return ((AG, RS), (RS, AG), (AG, AG))

    def totalTrafficTime(self, mesh: DeviceMesh):
        ta, da, tb, db = self._moving(mesh)
        total = 0.0
        for ka, kb in self._kinds():
            total += mesh.combine(ta / mesh.bws[ka][da], tb / mesh.bws[kb][db])
        return total / (mesh.shape[0] * mesh.shape[1])

    def totalLatency(self, mesh: DeviceMesh, K):
        ta, da, tb, db = self._moving(mesh)
        hop = (lambda n: n) if mesh.fabric == "ring" else (lambda n: min(n, 1))
        na, nb = hop(mesh.shape[da] - 1), hop(mesh.shape[db] - 1)
        total = 0.0
        for ka, kb in self._kinds():
            total += K * max(na * mesh.link_latencies[ka] + mesh.base_overheads[ka],
                             nb * mesh.link_latencies[kb] + mesh.base_overheads[kb])
        return total

    def pipelineOverhead(self, mesh: DeviceMesh, K):
        """Traffic of the first / last slice that no compute can hide (Autotuner.py:109-140):
        gathers of one pass overlap each other (max), a gather and a scatter do not (sum)."""
        ta, da, tb, db = self._moving(mesh)
        total = 0.0
        for ka, kb in self._kinds():
            a, b = ta / mesh.bws[ka][da], tb / mesh.bws[kb][db]
            total += mesh.combine(a, b) if ka == kb == "allgather" else a + b
        return total / (mesh.shape[0] * mesh.shape[1]) / K

    def emulate(self, mesh: DeviceMesh, K):
        B, I, O = self.bsize, self.in_dim, self.out_dim
        if getattr(mesh, "fused", None) is not None:
            OS, LS, RS = CostModel.Fused_OS, CostModel.Fused_LS, CostModel.Fused_RS
        else:
            OS, LS, RS = CostModel.MeshFlow_OS, CostModel.MeshFlow_LS, CostModel.MeshFlow_RS
        if not self.transpose:
            if self.dataflow == "os":
                t = (OS(mesh, B, O, I, K), LS(mesh, B, I, O, K), RS(mesh, I, O, B, K))
            elif self.dataflow == "ls":
                t = (LS(mesh, B, O, I, K), OS(mesh, B, I, O, K), RS(mesh, O, I, B, K))
            else:
                t = (RS(mesh, B, O, I, K), LS(mesh, I, B, O, K), OS(mesh, I, O, B, K))
        else:
            if self.dataflow == "os":
                t = (OS(mesh, O, B, I, K), RS(mesh, I, B, O, K), LS(mesh, O, I, B, K))
            elif self.dataflow == "ls":
                t = (RS(mesh, O, B, I, K), OS(mesh, I, B, O, K), LS(mesh, I, O, B, K))
            else:
                t = (LS(mesh, O, B, I, K), RS(mesh, B, I, O, K), OS(mesh, O, I, B, K))
        return sum(a + b for a, b in t)


class ComputeGraph:
    """Ordered dict-of-nodes IR (Autotuner.py:171-223)."""

    def __init__(self):
        self.nodenames: List[str] = []
        self.nodes: Dict[str, dict] = {}
        self.terminal = None

    def _new(self, op_type, inputs, shape, pos=None):
        for inp in inputs:
            assert inp in self.nodenames
        name = f"{op_type}:{len(self.nodes)}"
        if pos is None:
            self.nodenames.append(name)
        else:
            self.nodenames = self.nodenames[:pos] + [name] + self.nodenames[pos:]
        node = {"op_name": name, "op_type": op_type, "inputs": tuple(inputs), "shape": shape}
        self.nodes[name] = node
        self.terminal = node
        return node

    def add_operand(self, op_type, inputs, shape):
        return self._new(op_type, inputs, shape)

    def insert_operand(self, op_type, inputs, shape, pos):
        return self._new(op_type, inputs, shape, pos)

    def Input(self, shape):
        return self.add_operand("Input", (), list(shape))

    def FeedForward(self, input, output_dim):
        shape = copy.deepcopy(input["shape"])
        shape[-1] = output_dim
        return self.add_operand("FeedForward", (input["op_name"],), shape)

    def Attention(self, input, num_heads):
        shape = copy.deepcopy(input["shape"])
        assert shape[-1] % 3 == 0
        shape[-1] //= 3
        node = self.add_operand("Attention", (input["op_name"],), shape)
        node["num_heads"] = num_heads
        return node

    def Add(self, a, b):
        assert a["shape"] == b["shape"]
        return self.add_operand("Add", (a["op_name"], b["op_name"]), a["shape"])

    def Gelu(self, x):
        return self.add_operand("Gelu", (x["op_name"],), x["shape"])

    def LayerNorm(self, x):
        return self.add_operand("LayerNorm", (x["op_name"],), x["shape"])

    def printGraph(self):
        for n in self.nodenames:
            node = self.nodes[n]
            print("{}:{} = {}{}".format(n, node["shape"], node["op_type"], node["inputs"]))

    def ff_layers(self):
        """[(name, B, I, O)] of the FeedForward nodes in order."""
        out = []
        for n in self.nodenames:
            node = self.nodes[n]
            if node["op_type"] == "FeedForward":
                B = math.prod(node["shape"][:-1])
                I = self.nodes[node["inputs"][0]]["shape"][-1]
                out.append((n, B, I, node["shape"][-1]))
        return out


def build_transformerBlock(B, S, num_heads, head_dim, ffn_mult: int = 4):
    """The GPT block graph of the reference (Autotuner.py:225-240)."""
    g = ComputeGraph()
    dim = num_heads * head_dim
    x = g.Input([B, S, dim])
    n1 = g.LayerNorm(x)
    qkv = g.FeedForward(n1, 3 * dim)
    att = g.Attention(qkv, num_heads)
    proj = g.FeedForward(att, dim)
    a1 = g.Add(x, proj)
    n2 = g.LayerNorm(a1)
    f1 = g.FeedForward(n2, ffn_mult * dim)
    ge = g.Gelu(f1)
    f2 = g.FeedForward(ge, dim)
    a2 = g.Add(a1, f2)
    g.LayerNorm(a2)
    return g


def possibleK(B, I, O, meshshape, dataflow, blocksize: int = 8, max_k: int = 24):
    """Slice counts K >= 3 (or the only divisor) for which the sliced dimension splits into whole
    K x blocksize groups on both mesh axes (Autotuner.py:242-273 generalised to any block size)."""
    mlcm = math.lcm(meshshape[0], meshshape[1])
    dim = {"os": I, "ls": O}.get(dataflow, B)
    kdim = dim // mlcm // blocksize
    if kdim <= 0:
        return [1]
    ks = [k for k in range(3, max_k + 1) if kdim % k == 0]
    if not ks:
        ks = [k for k in (2, 1) if kdim % k == 0][:1] or [1]
    return ks


class Autotuner:
    """shapes: candidate mesh shapes, all with the same number of chips."""

    def __init__(self, graph: ComputeGraph, shapes, fabric: Optional[FabricConstants] = None, blocksize: int = 8,
                 matmul=None, verbose: bool = True, klist=None):
        self.graph, self.shapes = graph, list(shapes)
        self.fabric = fabric or FabricConstants.from_dict(TPUV4)
        self.blocksize, self.matmul, self.verbose = blocksize, matmul, verbose
        self.klist = klist
        self.transposition: Dict[str, bool] = {}
        self.dataflows: Dict[str, str] = {}
        # step 1: dataflow per FeedForward
        for name, B, I, O in graph.ff_layers():
            self.dataflows[name] = FFLayerModel(B, I, O).dataflow
        # step 2: transposition propagation
        pos = 0
        while pos < len(graph.nodenames):
            lname = graph.nodenames[pos]
            layer = graph.nodes[lname]
            t = layer["op_type"]
            if t == "Input":
                self.transposition[lname] = False
            elif t == "FeedForward":
                src = self.transposition[layer["inputs"][0]]
                self.transposition[lname] = (not src) if self.dataflows[lname] == "rs" else src
            elif t == "Add":
                a, b = layer["inputs"]
                ta, tb = self.transposition[a], self.transposition[b]
                if ta == tb:
                    self.transposition[lname] = ta
                else:
                    flip = a if ta else b          # bring the transposed operand back
                    keep = b if ta else a
                    tr = graph.insert_operand("Transpose", (flip,), layer["shape"], pos)
                    self.transposition[tr["op_name"]] = False
                    layer["inputs"] = (keep, tr["op_name"])
                    self.transposition[lname] = False
                    pos += 1
            else:
                self.transposition[lname] = self.transposition[layer["inputs"][0]]
            pos += 1
        self.ksplits: Dict[str, int] = {}
        self.bestshape = self.analyticalAutotune()

    def _log(self, *a):
        if self.verbose:
            print(*a)

    def _mesh(self, shape):
        return self.fabric.mesh(shape, matmul=self.matmul)

    def _ks(self, B, I, O, shape, dataflow):
        return list(self.klist) if self.klist else possibleK(B, I, O, shape, dataflow, self.blocksize)

    def analyticalAutotune(self):
        bestTime, bestMesh, bestks = float("inf"), self.shapes[0], {}
        for shape in self.shapes:
            mesh = self._mesh(shape)
            ks, traffic, latency, pipeline = {}, 0.0, 0.0, 0.0
            for name, B, I, O in self.graph.ff_layers():
                model = FFLayerModel(B, I, O, self.dataflows[name], self.transposition[name])
                traffic += model.totalTrafficTime(mesh)
                cand = self._ks(B, I, O, shape, self.dataflows[name])
                best = min(cand, key=lambda k: model.totalLatency(mesh, k) + 2 * model.pipelineOverhead(mesh, k))
                ks[name] = best
                latency += model.totalLatency(mesh, best)
                pipeline += model.pipelineOverhead(mesh, best)
            self._log("Mesh shape {}, traffic time {:.3f}, latency {:.3f}, pipeline: {:.3f} ms".format(
                shape, traffic * 1e3, latency * 1e3, pipeline * 1e3))
            if traffic + latency < bestTime:
                bestTime, bestMesh, bestks = traffic + latency, shape, ks
        self.ksplits = bestks
        self._report(bestMesh)
        return bestMesh

    def emulateFFTime(self, meshshape, sweep=False):
        mesh = self._mesh(meshshape)
        total, ks = 0.0, {}
        for name, B, I, O in self.graph.ff_layers():
            model = FFLayerModel(B, I, O, self.dataflows[name], self.transposition[name])
            cand = self._ks(B, I, O, meshshape, self.dataflows[name])
            bestK, bestT = cand[0], model.emulate(mesh, cand[0])
            for k in cand[1:]:
                t = model.emulate(mesh, k)
                if sweep:
                    self._log("FFtime at k={} is {}".format(k, t))
                if t < bestT:
                    bestK, bestT = k, t
                elif not sweep:
                    break
            total += bestT
            ks[name] = bestK
        self._log("FFtime: {}ms".format(total * 1e3))
        return total, ks

    def emulatedFinetune(self, sweep=False):
        self._log("Start emulated finetuning: ")
        idx = self.shapes.index(self.bestshape)
        cur_t, cur_k = self.emulateFFTime(self.bestshape)
        if sweep:
            for shp in self.shapes:
                t, k = self.emulateFFTime(shp, sweep=True)
                if t < cur_t:
                    cur_t, cur_k, self.bestshape = t, k, shp
            self.ksplits = cur_k
            self.predicted_time = cur_t
            self._report(self.bestshape)
            return self.bestshape
        def walk(i, t, k, step):
            while 0 <= i + step < len(self.shapes):
                t2, k2 = self.emulateFFTime(self.shapes[i + step])
                if t2 >= t:
                    break
                i, t, k = i + step, t2, k2
            return i, t, k
        lo = walk(idx, cur_t, cur_k, -1)
        hi = walk(idx, cur_t, cur_k, +1)
        best = min((lo, hi), key=lambda x: x[1])
        self.bestshape, self.predicted_time, self.ksplits = self.shapes[best[0]], best[1], best[2]
        self._report(self.bestshape)
        return self.bestshape

    def _report(self, shape):
        self._log("Best mesh shape is : {}".format(shape))
        for name in self.dataflows:
            self._log("Layer: {}\t Dataflow: {}\t Transpose: {}\t ksplit: {}".format(
                name, self.dataflows[name], self.transposition[name], self.ksplits.get(name)))

    def result(self) -> dict:
        return {"mesh": list(self.bestshape), "predicted_time_s": getattr(self, "predicted_time", None),
                "layers": [{"name": n, "dataflow": self.dataflows[n], "transpose": self.transposition[n],
                            "ksplit": self.ksplits.get(n)} for n in self.dataflows]}


def candidate_shapes(n_chips: int, min_dim: int = 1):
    """All R x C factorizations with both dimensions >= min_dim, rows ascending."""
    return [(r, n_chips // r) for r in range(min_dim, n_chips + 1)
            if n_chips % r == 0 and n_chips // r >= min_dim]


def main(argv=None):
    p = argparse.ArgumentParser(description="MeshSlice autotuner")
    p.add_argument("--ksplit", nargs=4, type=int, default=[8, 8, 8, 8])
    p.add_argument("--batchsize", type=int, default=-1, help="Default is number of chips")
    p.add_argument("--seqlen", type=int, default=2048)
    p.add_argument("--nheads", type=int, default=96)
    p.add_argument("--headdim", type=int, default=128)
    p.add_argument("--nrows", type=int, default=2)
    p.add_argument("--ncols", type=int, default=4)
    p.add_argument("--alg", type=str, default="noff")
    p.add_argument("--sweep", action="store_true")
    p.add_argument("--fabric-json", type=str, default="", help="constants fitted by BenchCollectives2D")
    p.add_argument("--fabric", type=str, default="b200", choices=["b200", "tpuv4"])
    p.add_argument("--netsim-config", type=str, default="",
                   help="fit the fabric constants from simulated sweeps of this system description "
                        "(a file, or the name of one shipped with the simulator)")
    p.add_argument("--netsim-topology", type=str, default="crossbar", help="crossbar or torus (one ring per mesh axis)")
    p.add_argument("--tuned-json", type=str, default="", help="write the decision here")
    p.add_argument("--meshes", type=str, nargs="*", default=[],
                   help="candidate mesh shapes RxC (default: every factorisation of nrows x ncols); one shape tunes "
                        "dataflows and slice counts for that mesh")
    p.add_argument("--blocksize", type=int, default=64)
    p.add_argument("--measure-matmul", action="store_true", help="time the tcgen05 GEMM instead of the analytic model")
    a = p.parse_args(argv)
    n = a.nrows * a.ncols
    B = n if a.batchsize <= 0 else a.batchsize
    graph = build_transformerBlock(B, a.seqlen, a.nheads, a.headdim)
    graph.printGraph()
    if a.netsim_config:
        from .utils import netsim
        fabric = FabricConstants.from_dict(netsim.fit_fabric(a.nrows, a.ncols, a.netsim_config, a.netsim_topology))
        print(f"fabric constants fitted from the simulator: {fabric.bws}")
    else:
        fabric = (FabricConstants.load(a.fabric_json) if a.fabric_json else
                  FabricConstants.from_dict(B200_NVSWITCH if a.fabric == "b200" else TPUV4))
    matmul = CostModel.MeasuredMatmul() if a.measure_matmul else None
    shapes = [tuple(int(v) for v in m.lower().split("x")) for m in a.meshes] or candidate_shapes(n)
    if any(len(sh) != 2 or sh[0] * sh[1] != n for sh in shapes):
        p.error(f"every --meshes entry must be RxC with R * C = {n}")
    print(shapes)
    tuner = Autotuner(graph, shapes, fabric=fabric, blocksize=a.blocksize, matmul=matmul,
                      klist=[1, 2, 4, 8] if a.fabric == "b200" and not a.fabric_json and not a.netsim_config else None)
    tuner.emulatedFinetune(a.sweep)
    if a.tuned_json:
        json.dump(tuner.result(), open(a.tuned_json, "w"), indent=1)
    return tuner


if __name__ == "__main__":
    main()
