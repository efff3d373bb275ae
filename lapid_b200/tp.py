"""Tensor parallelism for the quantized projections of a decoder layer (one process per GPU).

The reference has no multi-GPU code at all, so there is no interface to mirror; the parity statement
is "the sum of the shards' results equals the unsharded result".

* Column-parallel (q, k, v, gate, up): rank r owns weight rows ``[r*n/p, (r+1)*n/p)``. Rows of a
  lapid-quant matrix are independent block runs, so a shard is a byte range (the block formats: K-quants,
  MXFP4, i-quants) or a pair of plane slices (Int8, Int4). No communication; the outputs stay sharded and feed the row-parallel op.
* Row-parallel (o, down): rank r owns columns ``[r*k/p, (r+1)*k/p)``; ``k/p`` must be a multiple of
  the format's block length (256; 32 for Int8, Int4 and MXFP4) so shards are whole blocks, bit-identical to the unsharded ones. Shards are
  repacked once, at load, into a contiguous ``[n, k/p]`` matrix. Every rank produces a partial
  ``[M, n]`` f32 result and the partials are summed by an all-reduce.

Everything here works on numpy arrays (tests, CPU ranks over gloo) and on CUDA torch tensors.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

INT8, INT4, Q4_K, Q5_K, Q6_K, MXFP4 = 4, 5, 6, 7, 8, 9
IQ2_XXS, IQ2_S, IQ3_XXS, IQ2_XS = 10, 11, 12, 13
# array-of-structs formats: (elements, bytes) per block; Int8 and Int4 are planes of quants and f16 scales
_BLOCK = {Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), MXFP4: (32, 17),
          IQ2_XXS: (256, 66), IQ2_XS: (256, 74), IQ2_S: (256, 82), IQ3_XXS: (256, 98)}
_PLANES = {INT8: 1.0, INT4: 0.5}   # bytes of quants per element


def _known(fmt: int) -> None:
    if fmt not in _BLOCK and fmt not in _PLANES:
        raise ValueError(f"format {fmt} is not a quantized format of this backend")


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


def layout_total(fmt: int, n: int, k: int) -> int:
    _known(fmt)
    if fmt in _BLOCK:
        be, bb = _BLOCK[fmt]
        return _align(n * (k // be) * bb)
    return _align(_align(int(n * k * _PLANES[fmt])) + n * (k // 32) * 2)


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _zeros_like_bytes(x, nbytes: int):
    if _is_torch(x):
        import torch
        return torch.zeros(nbytes, dtype=torch.uint8, device=x.device)
    return np.zeros(nbytes, dtype=np.uint8)


def _pack(parts, total: int, like):
    """Concatenate byte pieces at their offsets into a zero-padded buffer of `total` bytes."""
    out = _zeros_like_bytes(like, total)
    for off, piece in parts:
        flat = piece.reshape(-1)
        out[off:off + flat.shape[0]] = flat
    return out


def check_divisible(fmt: int, n: int, k: int, world: int, kind: str) -> None:
    if kind == "column":
        if n % world:
            raise ValueError(f"column-parallel: n = {n} is not divisible by {world} ranks")
    else:
        _known(fmt)
        unit = _BLOCK[fmt][0] if fmt in _BLOCK else 32
        if k % (world * unit):
            raise ValueError(f"row-parallel: k = {k} must be a multiple of {world} x {unit}")


def shard_rows(fmt: int, q, n: int, k: int, rank: int, world: int):
    """Column-parallel shard: the quantized matrix of weight rows [rank*n/world, (rank+1)*n/world)."""
    check_divisible(fmt, n, k, world, "column")
    nl = n // world
    r0 = rank * nl
    if fmt in _BLOCK:
        be, bb = _BLOCK[fmt]
        rb = (k // be) * bb
        return _pack([(0, q[r0 * rb:(r0 + nl) * rb])], layout_total(fmt, nl, k), q), nl
    _known(fmt)
    rb = int(k * _PLANES[fmt])   # bytes of quants per weight row (Int4: a group's 32 nibbles are 16 consecutive bytes)
    so = _align(n * rb)
    kg = k // 32
    quants = q[r0 * rb:(r0 + nl) * rb]
    scales = q[so + r0 * kg * 2: so + (r0 + nl) * kg * 2]
    return _pack([(0, quants), (_align(nl * rb), scales)], layout_total(fmt, nl, k), q), nl


def shard_cols(fmt: int, q, n: int, k: int, rank: int, world: int):
    """Row-parallel shard: columns [rank*k/world, (rank+1)*k/world) of every weight row, repacked
    into a contiguous [n, k/world] lapid-quant matrix (whole blocks, bytes unchanged)."""
    check_divisible(fmt, n, k, world, "row")
    kl = k // world
    if fmt in _BLOCK:
        be, bb = _BLOCK[fmt]
        nb, nbl = k // be, kl // be
        blocks = q[:n * nb * bb].reshape(n, nb, bb)[:, rank * nbl:(rank + 1) * nbl, :]
        blocks = blocks.contiguous() if _is_torch(blocks) else np.ascontiguousarray(blocks)
        return _pack([(0, blocks)], layout_total(fmt, n, kl), q), kl
    _known(fmt)
    rb, rbl = int(k * _PLANES[fmt]), int(kl * _PLANES[fmt])   # (shards are whole 32-element groups, so also whole bytes of Int4)
    so = _align(n * rb)
    kg, kgl = k // 32, kl // 32
    quants = q[:n * rb].reshape(n, rb)[:, rank * rbl:(rank + 1) * rbl]
    scales = q[so:so + n * kg * 2].reshape(n, kg, 2)[:, rank * kgl:(rank + 1) * kgl, :]
    if _is_torch(q):
        quants, scales = quants.contiguous(), scales.contiguous()
    else:
        quants, scales = np.ascontiguousarray(quants), np.ascontiguousarray(scales)
    return _pack([(0, quants), (_align(n * rbl), scales)], layout_total(fmt, n, kl), q), kl


# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LayerShape:
    """Projection shapes of one Llama-architecture decoder layer."""
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int

    def projections(self):
        """(name, n, k, parallel kind) in execution order."""
        d, kv = self.d_model, self.n_kv_heads * self.head_dim
        return [("q", self.n_heads * self.head_dim, d, "column"), ("k", kv, d, "column"), ("v", kv, d, "column"),
                ("o", d, self.n_heads * self.head_dim, "row"), ("gate", self.ffn, d, "column"),
                ("up", self.ffn, d, "column"), ("down", d, self.ffn, "row")]


LLAMA3_8B = LayerShape(4096, 32, 8, 128, 14336)
LLAMA_70B = LayerShape(8192, 64, 8, 128, 28672)


def use_more_bits(i: int, n_layers: int) -> bool:
    """Which layers get the wider format in a Q4_K_M-style mix
    (crates/lapid-convert/src/policy.rs:154-157): the first and last eighth and every third between."""
    return i < n_layers // 8 or i >= 7 * n_layers // 8 or (i - n_layers // 8) % 3 == 2


def q4km_format(name: str, layer: int, n_layers: int) -> int:
    """Q6_K for attn_v and for ffn_down in the `use_more_bits` layers, Q4_K elsewhere."""
    if name == "v":
        return Q6_K
    if name == "down" and use_more_bits(layer, n_layers):
        return Q6_K
    return Q4_K


def local_shape(name: str, n: int, k: int, kind: str, world: int):
    return (n // world, k) if kind == "column" else (n, k // world)


class TpLayer:
    """One decoder layer's quantized projections on this rank.

    `matmul(fmt, x, w, n, k)` is injected: the CUDA backend on a GPU rank, the CPU oracle in the
    gloo tests. `all_reduce(t)` sums a partial result over the ranks in place (identity at world 1).
    The attention mixing itself is outside this path: q's output feeds o directly, which keeps the
    dependency chain and the sharding (q's columns are o's k shard) of the real layer.
    """

    def __init__(self, shape: LayerShape, weights: dict, formats: dict, world: int, matmul, all_reduce, ops):
        self.shape, self.w, self.fmt, self.world = shape, weights, formats, world
        self.matmul, self.all_reduce, self.ops = matmul, all_reduce, ops
        self.dims = {name: local_shape(name, n, k, kind, world) for name, n, k, kind in shape.projections()}

    def _mm(self, name, x):
        n, k = self.dims[name]
        return self.matmul(self.fmt[name], x, self.w[name], n, k)

    def forward(self, h):
        ops = self.ops
        x = ops.rms_normalise(h)
        q = self._mm("q", x)
        self._mm("k", x)
        self._mm("v", x)
        o = self._mm("o", q)                      # partial sums over this rank's k shard
        self.all_reduce(o)
        h = ops.add(h, o)
        x = ops.rms_normalise(h)
        g = self._mm("gate", x)
        u = self._mm("up", x)
        d = self._mm("down", ops.silu_mul(g, u))  # partial
        self.all_reduce(d)
        return ops.add(h, d)


class NumpyOps:
    @staticmethod
    def rms_normalise(x):
        x = np.asarray(x, np.float32)
        return (x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True) + 1e-6)).astype(np.float32)

    @staticmethod
    def add(a, b):
        return (np.asarray(a, np.float32) + np.asarray(b, np.float32)).astype(np.float32)

    @staticmethod
    def silu_mul(g, u):
        g = np.asarray(g, np.float64)
        return (g / (1.0 + np.exp(-g)) * np.asarray(u, np.float64)).astype(np.float32)


class TorchOps:
    """The few elementwise steps between projections, on CUDA tensors (plumbing, not the product)."""

    @staticmethod
    def rms_normalise(x):
        import torch
        return x * torch.rsqrt(x.float().pow(2).mean(dim=-1, keepdim=True) + 1e-6)

    @staticmethod
    def add(a, b):
        return a + b

    @staticmethod
    def silu_mul(g, u):
        import torch
        return torch.nn.functional.silu(g) * u


class PeerAllReduce:
    """The library's one-shot all-reduce over peer-mapped memory (`lapid_b200_tp_all_reduce`).

    torch's symmetric-memory allocator supplies the buffer that every rank can address (plumbing);
    the kernel that moves and sums the data is the library's own. Used for decode-sized results;
    larger ones (prefill) stay on NCCL, whose ring moves 2x the data instead of world x.
    """

    def __init__(self, backend, rank: int, world: int, device, group=None, max_elems: int = 65536):
        import ctypes as C
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        self.backend, self.max_elems, self._lib = backend, max_elems, _lib
        lib = _lib.lib()
        nbytes = int(lib.lapid_b200_tp_comm_bytes(world, max_elems))
        self.mem = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.mem, group if group is not None else dist.group.WORLD)
        self.mem.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        ptrs = (C.c_void_p * world)(*[int(p) for p in self.handle.buffer_ptrs])
        h = C.c_void_p()
        _lib.check(lib.lapid_b200_tp_comm_create(backend._h, rank, world, ptrs, max_elems, C.byref(h)))
        self._h = h

    def fits(self, numel: int) -> bool:
        return numel % 4 == 0 and numel <= self.max_elems

    def __call__(self, buf, numel: int) -> None:
        self._lib.check(self._lib.lib().lapid_b200_tp_all_reduce(self._h, buf._h, 0, numel))

    def pushing(self, launch, buffers):
        """A zero-argument callable that queues `launch` (one decode MatMul) so that its result goes
        to every rank's slots from the GEMV's own epilogue (`lapid_b200_tp_matmul_push`); follow it
        with `rms_norm`, which sums the ranks' partials while it normalises."""
        arr, bufs = self.backend._pack([launch], buffers)
        fn, check, h, nb = self._lib.lib().lapid_b200_tp_matmul_push, self._lib.check, self._h, len(buffers)

        def run():
            check(fn(h, arr, bufs, nb))
        run.keep = (arr, bufs, list(buffers))
        return run

    def rms_norm(self, out, rows: int, cols: int, eps: float = 1e-6, residual=None, weight=None, sum_out=None, qact=None,
                 layout: int = 0) -> None:
        """`Backend.rms_norm` with x = the sum over ranks of the push in progress (`lapid_b200_tp_rms_norm_act`)."""
        h = lambda b: b._h if b is not None else None
        self._lib.check(self._lib.lib().lapid_b200_tp_rms_norm_act(self._h, h(residual), h(weight), h(sum_out), out._h, rows, cols, eps,
                                                                   h(qact), layout))

    def close(self):
        if self._h:
            self._lib.lib().lapid_b200_tp_comm_free(self._h)
            self._h = None


def d_model_of(shape) -> int:
    return shape.d_model


class GpuTpLayers:
    """A stack of decoder layers' projections on one GPU rank, driven through the C ABI.

    Buffers are allocated once (torch tensors wrapped as library buffers); a token step queues, per
    layer, four launch lists -- [q, k, v], [o], [gate, up], [down] -- on the current torch stream with
    `execute_async`, the normalise / residual / SwiGLU steps with the library's two glue kernels, and
    the two all-reduces of the row-parallel outputs with the library's peer all-reduce (or NCCL
    through torch.distributed). The whole step can be captured in a CUDA graph.
    """

    def __init__(self, backend, shape: LayerShape, world: int, rank: int, m: int, weights: list, formats: list,
                 group=None, peer_all_reduce=None, fused: bool = False, fuse_act: bool = True, skip_collective: bool = False):
        import torch
        from .backend import matmul_launch
        self.be, self.shape, self.world, self.rank, self.m, self.group = backend, shape, world, rank, m, group
        self.peer = peer_all_reduce
        self.skip_collective = skip_collective   # timing only: the exchanges are left out (the results are then wrong)
        # fused: the row-parallel GEMVs push their partials from their epilogue and the following
        # rms_norm sums them: the all-reduce has no kernel of its own
        self.fused = bool(fused and peer_all_reduce is not None and world > 1 and peer_all_reduce.fits(m * d_model_of(shape)))
        dev = weights[0]["q"].device
        d = shape.d_model
        proj = {name: local_shape(name, n, k, kind, world) for name, n, k, kind in shape.projections()}
        f32 = dict(dtype=torch.float32, device=dev)
        self.h = torch.zeros(m, d, **f32)
        self.x = torch.zeros(m, d, **f32)
        self.outs = {name: torch.zeros(m, proj[name][0], **f32) for name in proj}
        self.act = torch.zeros(m, proj["gate"][0], **f32)
        torch.cuda.synchronize(dev)
        wrap = backend.wrap_tensor
        self.out_bufs = {name: wrap(self.outs[name]) for name in ("o", "down")}
        self.hw = torch.zeros(m, d, **f32)
        torch.cuda.synchronize(dev)
        self._glue = {"h": wrap(self.h), "hw": wrap(self.hw), "x": wrap(self.x), "o": self.out_bufs["o"],
                      "down": self.out_bufs["down"], "gate": wrap(self.outs["gate"]), "up": wrap(self.outs["up"]),
                      "act": wrap(self.act)}
        self._keep = []
        self.steps = []
        # fuse_act: the glue kernels also write x and act as the quantized operand of the decode GEMVs that
        # read them (no pre-pass kernel in front of q/k/v, gate/up and down); per layer, the layout of the
        # phase's first projection is used, a projection that wants another one keeps the f32 operand
        self.fuse_act = bool(fuse_act and m <= 8)
        self.qx = torch.zeros(2 * m * d + 2 * d + 4096, dtype=torch.uint8, device=dev)
        self.qact = torch.zeros(2 * m * proj["gate"][0] + 2 * proj["gate"][0] + 4096, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize(dev)
        self._glue["qx"], self._glue["qact"] = wrap(self.qx), wrap(self.qact)
        self.act_layouts = []   # per weight set: layout codes for (q/k/v phase, gate/up phase, down), None = not fused
        for w, f in zip(weights, formats):
            bufs = [wrap(self.x), wrap(self.outs["q"]), wrap(self.act)]                 # 0 x, 1 q_out, 2 act
            order = ["q", "k", "v", "o", "gate", "up", "down"]
            bufs += [wrap(w[n_]) for n_ in order]                                       # 3..9 weights
            bufs += [wrap(self.outs[n_]) for n_ in order]                               # 10..16 outputs
            bufs += [wrap(self.qx), wrap(self.qact)]                                    # 17 quantized x, 18 quantized act
            idx = {n_: i for i, n_ in enumerate(order)}

            def launch(name, a_id, quantized=False):
                n, k = proj[name]
                return matmul_launch(f[name], m, n, k, inputs=(a_id, 3 + idx[name]), output=10 + idx[name], a_quantized=quantized)

            def layout_of(name, holder):
                if not self.fuse_act:
                    return None
                try:
                    lay, nbytes = backend.act_layout(launch(name, 0))
                except Exception:
                    return None
                return lay if nbytes <= holder.numel() else None

            def phase(names, f32_id, q_id, holder):
                lay = layout_of(names[0], holder)
                ls = [launch(n_, q_id, True) if lay is not None and layout_of(n_, holder) == lay else launch(n_, f32_id) for n_ in names]
                return lay, ls

            lay_qkv, l_qkv = phase(["q", "k", "v"], 0, 17, self.qx)
            lay_gu, l_gu = phase(["gate", "up"], 0, 17, self.qx)
            lay_down, l_down = phase(["down"], 2, 18, self.qact)
            self.act_layouts.append((lay_qkv, lay_gu, lay_down))
            lists = [l_qkv, [launch("o", 1)], l_gu, l_down]
            backend.prepare([l for ls in lists for l in ls])
            step = [backend.packed(ls, bufs) for ls in lists]
            if self.fused:
                step[1] = self.peer.pushing(lists[1][0], bufs)
                step[3] = self.peer.pushing(lists[3][0], bufs)
            self.steps.append(step)
            self._keep.append(bufs)

    def all_reduce(self, name):
        if self.world == 1 or self.skip_collective:
            return
        t = self.outs[name]
        if self.peer is not None and self.peer.fits(t.numel()):
            self.peer(self.out_bufs[name], t.numel())
        else:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)

    def _q_of(self, layout, holder):
        """Keyword arguments that make a glue call write the quantized operand too."""
        return {} if layout is None else {"qact": self._glue[holder], "layout": layout}

    def _attention_half(self, i: int, res):
        """q, k, v, then o and its exchange: hw = res + sum over ranks of o; x = norm(hw), quantized for gate / up."""
        be, m, d, w = self.be, self.m, self.shape.d_model, self._glue
        qkv, o, _, _ = self.steps[i % len(self.steps)]
        lay_gu = self.act_layouts[i % len(self.steps)][1]
        qkv()
        o()
        if self.fused:
            self.peer.rms_norm(w["x"], m, d, residual=res, sum_out=w["hw"], **self._q_of(lay_gu, "qx"))
        else:
            self.all_reduce("o")
            be.rms_norm(w["o"], w["x"], m, d, residual=res, sum_out=w["hw"], **self._q_of(lay_gu, "qx"))    # h' = h + o;    x = norm(h')

    def _ffn_half(self, i: int):
        """gate, up, SwiGLU, then down and its exchange: hw += sum over ranks of down; x = norm(hw) for the next layer."""
        be, m, d, w = self.be, self.m, self.shape.d_model, self._glue
        sets = len(self.steps)
        _, _, gu, down = self.steps[i % sets]
        lay_down = self.act_layouts[i % sets][2]
        lay_next = self.act_layouts[(i + 1) % sets][0]
        gu()
        be.silu_mul(w["gate"], w["up"], w["act"], self.act.numel(), rows=m, **self._q_of(lay_down, "qact"))
        down()
        if self.fused:
            self.peer.rms_norm(w["x"], m, d, residual=w["hw"], sum_out=w["hw"], **self._q_of(lay_next, "qx"))
        else:
            self.all_reduce("down")
            be.rms_norm(w["down"], w["x"], m, d, residual=w["hw"], sum_out=w["hw"], **self._q_of(lay_next, "qx"))  # h'' = h' + down; x = norm(h'') for the next layer

    def token(self, n_layers: int):
        """Queues `n_layers` layer steps (cycling over the distinct weight sets) on the current stream.

        Between the projections only the library's two glue kernels run: `rms_norm` (with the
        residual add folded in) and `silu_mul`. The residual stream of the token starts from `self.h`
        (left untouched, so a captured graph replays the same token) and ends in `self.h_out`."""
        w = self._glue
        self.be.rms_norm(w["h"], w["x"], self.m, self.shape.d_model, **self._q_of(self.act_layouts[0][0], "qx"))  # x = norm(h)
        for i in range(n_layers):
            self._attention_half(i, w["h"] if i == 0 else w["hw"])
            self._ffn_half(i)
        self.h_out = self.hw
        return self.hw

    def first_row_parallel(self):
        """Queues the first layer up to and including its first exchange and returns `h + sum over ranks of o`:
        the first row-parallel result, whose inputs are the same however the layer is sharded."""
        w = self._glue
        self.be.rms_norm(w["h"], w["x"], self.m, self.shape.d_model, **self._q_of(self.act_layouts[0][0], "qx"))
        self._attention_half(0, w["h"])
        return self.hw
