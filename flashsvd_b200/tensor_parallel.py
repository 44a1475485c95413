"""Tensor-parallel decode of one model over the GPUs of a node (one process per GPU).

Partitioning (configuration 4 of the benchmark, the Llama-2-70B shape): every rank takes H / N
query heads with their Hk / N key / value heads and I / N columns of the SwiGLU intermediate:

    sharded by rows      q_u, k_u, v_u (the rank's heads), gate_u, up_u (the rank's slice of I)
    sharded by columns   o_v (inputs = the rank's heads), down_v (inputs = the rank's slice of I)
    replicated           q_v, k_v, v_v, gate_v, up_v (they read the full hidden state), o_u, down_u

so that every rank produces a partial sum [B, d] of the attention output projection and of the MLP
output, and two exchanges per layer complete them.  The KV cache of a rank holds its own heads only.

Two ways to run a layer:

``exchange="peer"`` (default for bf16): ``fsvd_tp_decode_layer`` — the layer as tiled tensor-core
    GEMMs on the shards; the epilogue of the o lift and of the down lift stores every finished tile
    into an exchange region of EVERY rank (peer stores over NVLink, regions mapped with CUDA IPC) and
    raises a flag per CTA; the next kernel polls the flags of its own region, adds the partial sums
    in rank order plus the residual and applies the next RMSNorm.  No collective call on the path.
``exchange="nccl"``: the library's per-op entry points on the shards (``fsvd_qkv_rope_append``,
    ``fsvd_flash_decode``, ``fsvd_lowrank_proj``, ``fsvd_mlp_swiglu_decode``) with
    ``torch.distributed.all_reduce`` of the two partial sums; rank 0 adds the residual before the
    all-reduce, so the sum carries it once.  The baseline the peer exchange is measured against.

Rounding differs from the single-GPU path in one place: each rank's partial output is rounded to
the model dtype before the sum (the single-GPU path rounds the rank-space vector once, after the
full sum).

Reference: the partitioning is the one the reference's north-star configuration names; its own code
has no tensor-parallel path (it shards whole layers with ``layer_device_map``,
runtime/cache/attn_dense_kv.py:52-58).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import check

ROW_SHARDED = ("q_u", "k_u", "v_u", "gate_u", "up_u")
COL_SHARDED = ("o_v", "down_v")


def shard_ranges(H: int, Hk: int, Dh: int, I: int, rank: int, world: int):
    """(query rows, key/value rows, intermediate columns) of ``rank`` as slices."""
    if H % world or Hk % world or I % world or (I // world) % 8:
        raise ValueError(f"H={H}, Hk={Hk} and I={I} must split evenly over {world} ranks (I / ranks a multiple of 8)")
    hq, hk, ii = H // world * Dh, Hk // world * Dh, I // world
    return slice(rank * hq, (rank + 1) * hq), slice(rank * hk, (rank + 1) * hk), slice(rank * ii, (rank + 1) * ii)


def shard_layer_weights(w: dict, *, H: int, Hk: int, Dh: int, rank: int, world: int) -> dict:
    """The rank's view of one layer's factors (keys as in the oracle: q_v .. down_u, ln1, ln2)."""
    I = w["gate_u"].shape[0]
    sq, sk, si = shard_ranges(H, Hk, Dh, I, rank, world)
    out = dict(w)
    out["q_u"], out["k_u"], out["v_u"] = w["q_u"][sq], w["k_u"][sk], w["v_u"][sk]
    out["o_v"] = w["o_v"][:, sq]
    out["gate_u"], out["up_u"] = w["gate_u"][si], w["up_u"][si]
    out["down_v"] = w["down_v"][:, si]
    return {k: (v.contiguous() if torch.is_tensor(v) else v) for k, v in out.items()}


def _rendezvous() -> None:
    """Host barrier of the ranks with the device idle on both sides."""
    torch.cuda.synchronize()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
        torch.cuda.synchronize()


def _all_reduce(t: torch.Tensor) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t)
    return t


def region_layout(world: int, max_rows: int, d: int) -> dict:
    """Byte offsets inside an exchange region (mirror of csrc/fsvd_exchange.h): flags
    [2 parities][world][flag_cap] uint32 at ``flags``, slots [2 parities][world][slot_bytes] at
    ``slots`` (a slot = one rank's partial sums, bf16 [rows, d])."""
    al = lambda n: (n + 255) // 256 * 256
    flag_cap = (d + 127) // 128 * 8
    slot_bytes = al(max_rows * d * 2)
    flags = 256
    slots = flags + al(2 * world * flag_cap * 4)
    return {"flag_cap": flag_cap, "slot_bytes": slot_bytes, "flags": flags, "slots": slots,
            "total": slots + 2 * world * slot_bytes}


class PeerExchange:
    """This rank's exchange region, the other ranks' regions mapped into this process, and the
    library's exchange object over them (``handle``).

    ``regions=None``: the region is allocated by the library, its 64-byte export handle is gathered
    over ``group`` (any backend) and the peers' regions are imported; ranks must be the processes
    of one node with peer access between their GPUs.  ``regions=[...]``: base addresses given by
    the caller (tests on one GPU)."""

    def __init__(self, *, rank: int, world: int, max_rows: int, d: int, group=None, regions=None):
        lib = _lib.load()
        self.rank, self.world, self.group = int(rank), int(world), group
        self.nbytes = int(lib.fsvd_exchange_region_bytes(self.world, int(max_rows), int(d)))
        if self.nbytes == 0:
            raise ValueError(f"exchange of {world} ranks, {max_rows} rows, width {d}: at most 8 ranks, 128 rows")
        self._own, self._imported, self.handle, self._trace = None, [], None, None
        if regions is None:
            p = C.c_void_p()
            check(lib.fsvd_exchange_region_alloc(self.nbytes, C.byref(p)))
            self._own = p.value
            mine = C.create_string_buffer(64)
            check(lib.fsvd_exchange_region_export(self._own, mine))
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(mine.raw), group=group)   # also: every region exists and is zero
            regions = []
            for q in range(self.world):
                if q == self.rank:
                    regions.append(self._own)
                    continue
                pp = C.c_void_p()
                check(lib.fsvd_exchange_region_import(handles[q], C.byref(pp)))
                self._imported.append(pp.value)
                regions.append(pp.value)
        self.regions = [int(r) for r in regions]
        arr = (C.c_void_p * self.world)(*self.regions)
        h = C.c_void_p()
        check(lib.fsvd_exchange_create(self.rank, self.world, arr, int(max_rows), int(d),
                                       torch.cuda.current_stream().cuda_stream, C.byref(h)))
        self.handle = h

    def start_trace(self, records: int = 4096) -> None:
        """Record the timing of every reduction from now on (before the first layer call to be traced;
        launches already captured into a CUDA graph keep their setting)."""
        self._trace = torch.zeros(int(records), 3, dtype=torch.int64, device=torch.cuda.current_device())
        check(_lib.load().fsvd_exchange_set_trace(self.handle, self._trace.data_ptr(), self._trace.numel() * 8))

    def trace_summary(self) -> dict:
        """Of the traced reductions: microseconds between the rank's own GEMM finishing and all ranks'
        flags being seen (``wait``: peers' lateness + the transfer), and of the reduction itself."""
        if self._trace is None:
            return {"exchanges": 0}
        t = self._trace.cpu()
        t = t[(t > 0).all(dim=1)]
        if t.numel() == 0:
            return {"exchanges": 0}
        wait, red = (t[:, 1] - t[:, 0]).double() / 1e3, (t[:, 2] - t[:, 1]).double() / 1e3
        q = lambda v, p: float(torch.quantile(v, p))
        return {"exchanges": int(t.shape[0]), "wait_us_median": q(wait, 0.5), "wait_us_p90": q(wait, 0.9),
                "wait_us_max": float(wait.max()), "reduce_us_median": q(red, 0.5)}

    def close(self) -> None:
        """Collective when the regions were exchanged over a group: no rank unmaps while another may
        still be storing into its region."""
        lib = _lib.load()
        if self.handle is not None:
            torch.cuda.synchronize()
            if self._own is not None and self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            lib.fsvd_exchange_destroy(self.handle)
            self.handle = None
            for p in self._imported:
                lib.fsvd_exchange_region_release(p)
            self._imported = []
            if self._own is not None:
                if self.world > 1 and dist.is_initialized():
                    dist.barrier(group=self.group)
                lib.fsvd_exchange_region_free(self._own)
                self._own = None


class TPDecodeLayer:
    """One decoder layer on this rank's shards.  ``exchange``: a PeerExchange (partial sums exchanged
    inside the kernels) or None (per-op entry points + NCCL all-reduce)."""

    def __init__(self, w_shard: dict, *, H: int, Hk: int, Dh: int, rank: int, world: int, batch: int, S_max: int,
                 eps: float, device, dtype=torch.bfloat16, exchange: PeerExchange | None = None):
        self.exchange = exchange
        if exchange is not None:
            if dtype != torch.bfloat16 or not 1 <= batch <= 128:
                raise ValueError("the peer-exchange layer takes bf16 and 1..128 sequences")
        elif batch > (8 if dtype == torch.bfloat16 else 4):
            raise ValueError("the all-reduce layer takes the batch sizes of the single-launch kernel (<= 8)")
        self.rank, self.world, self.eps = int(rank), int(world), float(eps)
        self.Hl, self.Hkl, self.Dh = H // world, Hk // world, Dh

        def dev(t):
            return t.detach().to(device=device, dtype=dtype).contiguous()

        w = w_shard
        self.ln1, self.ln2 = dev(w["ln1"]), dev(w["ln2"])
        self.qkv_v = dev(torch.cat([w["q_v"], w["k_v"], w["v_v"]], 0))
        self.q_u, self.k_u, self.v_u = dev(w["q_u"]), dev(w["k_u"]), dev(w["v_u"])
        self.o_v, self.o_u = dev(w["o_v"]), dev(w["o_u"])
        self.upgate_v = dev(torch.cat([w["up_v"], w["gate_v"]], 0))
        self.gate_u, self.up_u = dev(w["gate_u"]), dev(w["up_u"])
        self.down_v, self.down_u = dev(w["down_v"]), dev(w["down_u"])
        self.ranks = (w["q_u"].shape[1], w["k_u"].shape[1], w["v_u"].shape[1])
        self.k_cache = torch.zeros(batch, S_max, self.Hkl, Dh, dtype=dtype, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        d, Il = self.o_u.shape[0], self.gate_u.shape[0]
        dims = ops.make_dims(dtype=dtype, B=batch, d=d, H=self.Hl, Hk=self.Hkl, Dh=Dh, I=Il, Rq=self.ranks[0],
                             Rk=self.ranks[1], Rv=self.ranks[2], Ro=self.o_v.shape[0], Rg=self.gate_u.shape[1],
                             Ru=self.up_u.shape[1], Rd=self.down_v.shape[0], S_max=S_max, eps=eps)
        self.dims = dims
        if exchange is None:
            self.ws = ops.make_workspace(dims, device)
        else:
            self.ws = ops.make_tp_workspace(dims, device)
            self.out = torch.empty(batch, d, dtype=dtype, device=device)
            self.out_norm = torch.empty(batch, d, dtype=dtype, device=device)   # rmsnorm(out) . the next norm weight
            self._struct = ops.make_layer_struct({
                "ln1_w": self.ln1, "qkv_v": self.qkv_v, "q_u": self.q_u, "k_u": self.k_u, "v_u": self.v_u, "o_v": self.o_v,
                "o_u": self.o_u, "ln2_w": self.ln2, "upgate_v": self.upgate_v, "gate_u": self.gate_u, "up_u": self.up_u,
                "down_v": self.down_v, "down_u": self.down_u, "k_cache": self.k_cache, "v_cache": self.v_cache})

    def bytes_per_step(self, ctx: int, batch: int) -> int:
        """Factor bytes this rank streams per step plus the K / V rows it reads."""
        fac = sum(t.numel() * t.element_size() for t in (self.qkv_v, self.q_u, self.k_u, self.v_u, self.o_v, self.o_u,
                                                         self.upgate_v, self.gate_u, self.up_u, self.down_v, self.down_u))
        return fac + 2 * batch * ctx * self.Hkl * self.Dh * self.k_cache.element_size()

    def forward(self, x: torch.Tensor, seqlens: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, x_norm=None,
                next_norm_w=None) -> torch.Tensor:
        """Peer exchange only: ``x_norm`` = ln1-normalised x the caller holds (``out_norm`` of the
        layer before); ``next_norm_w``: also leave rmsnorm(output) * next_norm_w in ``self.out_norm``."""
        B = x.shape[0]
        if self.exchange is not None:
            if B != self.dims.B:
                raise ValueError(f"the layer was built for {self.dims.B} sequences")
            return ops.tp_decode_layer(self.dims, self._struct, cos, sin, seqlens, x, self.out, self.exchange.handle, self.ws,
                                       x_norm_in=x_norm, next_norm_w=next_norm_w,
                                       x_norm_out=self.out_norm if next_norm_w is not None else None)
        if x_norm is not None or next_norm_w is not None:
            raise ValueError("x_norm / next_norm_w belong to the peer-exchange layer")
        first = self.rank == 0
        q = ops.qkv_rope_append(x, self.qkv_v, self.q_u, self.k_u, self.v_u, cos, sin, self.k_cache, self.v_cache,
                                seqlens, self.ws, num_heads=self.Hl, num_kv_heads=self.Hkl, head_dim=self.Dh,
                                ranks=self.ranks, norm_w=self.ln1, eps=self.eps)
        a = ops.flash_decode(q, self.k_cache, self.v_cache, seqlens, self.ws, seqlen_add=1)
        h = ops.lowrank_proj(a.view(B, self.Hl * self.Dh), self.o_v, self.o_u, self.ws, residual=x if first else None)
        _all_reduce(h)                                   # partial sums of the output projection
        y = ops.mlp_swiglu_decode(h, self.gate_u, self.up_u, self.down_v, self.down_u, self.ws, upgate_v=self.upgate_v,
                                  norm_w=self.ln2, eps=self.eps, residual=h if first else None)
        return _all_reduce(y)                            # partial sums of the down projection


class TPModel:
    """Whole-model tensor-parallel decode: replicated embedding, final norm and lm_head, sharded
    layers.  One step = embed -> layers (two all-reduces each) -> norm -> lm_head -> argmax; the
    step is captured into a CUDA graph (kernels and NCCL collectives) on first use and replayed.
    Tokens and sequence lengths stay on the device."""

    def __init__(self, layers, embed, final_norm, lm_head, *, batch: int, S_max: int, head_dim: int, theta: float,
                 eps: float, device, dtype=torch.bfloat16, use_graph: bool = True):
        from .engine import rope_tables

        if batch > (8 if dtype == torch.bfloat16 else 4):
            raise ValueError("the model step (replicated lm_head through fsvd_lift) takes at most 8 sequences; "
                             "TPDecodeLayer with a PeerExchange takes up to 128")
        self.layers, self.embed, self.final_norm, self.lm_head = layers, embed, final_norm, lm_head
        self.B, self.S_max, self.eps, self.device, self.dtype = int(batch), int(S_max), float(eps), device, dtype
        self.cos, self.sin = rope_tables(self.S_max, head_dim, theta, dtype, device)
        self.tokens = torch.zeros(self.B, dtype=torch.int64, device=device)
        self.seqlens = torch.zeros(self.B, dtype=torch.int32, device=device)
        self.logits = torch.zeros(self.B, embed.shape[0], dtype=dtype, device=device)
        dims = ops.make_dims(dtype=dtype, B=self.B, d=embed.shape[0], Ro=embed.shape[1])
        self._head_ws = ops.make_workspace(dims, device)
        self._graph = None
        self._use_graph = bool(use_graph)
        self._x0 = torch.zeros(self.B, embed.shape[1], dtype=dtype, device=device)

    def _step_eager(self) -> None:
        x = torch.index_select(self.embed, 0, self.tokens, out=self._x0)
        if self.layers and self.layers[0].exchange is not None:
            # the kernel that finishes a layer also applies the next layer's input norm (the final
            # norm after the last layer)
            xn = None
            for i, layer in enumerate(self.layers):
                nxt = self.layers[i + 1].ln1 if i + 1 < len(self.layers) else self.final_norm
                x = layer.forward(x, self.seqlens, self.cos, self.sin, x_norm=xn, next_norm_w=nxt)
                xn = layer.out_norm
        else:
            for layer in self.layers:
                x = layer.forward(x, self.seqlens, self.cos, self.sin)
            xf = x.float()
            xn = self.final_norm * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(self.dtype)
        ops.lift(xn, self.lm_head, self._head_ws, out=self.logits)
        self.tokens.copy_(self.logits.float().argmax(-1))
        self.seqlens.add_(1)

    def step(self, n: int = 1) -> None:
        for _ in range(int(n)):
            if not self._use_graph:
                self._step_eager()
                continue
            if self._graph is None:
                # one eager step first (workspaces, cached programs, NCCL communicators), undone below;
                # the ranks start it together: a wait for a peer's partial sums is bounded by the
                # library's wait budget (about 2 s), which a rank still building its model would exceed
                tok, sl = self.tokens.clone(), self.seqlens.clone()
                _rendezvous()
                self._step_eager()
                torch.cuda.synchronize()
                self.tokens.copy_(tok)
                self.seqlens.copy_(sl)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step_eager()
                self._graph = g
                self.tokens.copy_(tok)
                self.seqlens.copy_(sl)
                _rendezvous()
                # the captured step has not run: positions written by the eager step are rewritten
            self._graph.replay()

    exchange = None

    def close(self) -> None:
        """Collective: releases the graph and the exchange regions."""
        self._graph = None
        if self.exchange is not None:
            self.exchange.close()
            self.exchange = None

    def status(self) -> int:
        for layer in self.layers:
            st = layer.ws.status()
            if st:
                return st
        return 0

    def bytes_per_step(self, ctx: int) -> int:
        """Algorithmic bytes this rank reads per step (its factor shards, replicated factors, its K / V
        rows, lm_head)."""
        return sum(l.bytes_per_step(ctx, self.B) for l in self.layers) + self.lm_head.numel() * self.lm_head.element_size()


def random_tp_model(shape, *, rank: int, world: int, device, batch: int, ctx: int, max_new: int, seed: int = 0,
                    dtype=torch.bfloat16, n_layers=None, use_graph: bool = True, exchange: str = "peer",
                    shard_of: int | None = None, trace: bool = False) -> TPModel:
    """Seeded random model of ``shape`` (a synthetic.ModelShape), every rank drawing the same full
    factors on its device and keeping its shards; caches pre-filled with ``ctx`` N(0,1) rows.
    ``exchange``: "peer" (partial sums exchanged inside the kernels) or "nccl" (all-reduce).
    ``shard_of`` (profiling on one GPU): the weights are rank 0's share of a partition over
    ``shard_of`` ranks while the exchange has the ``world`` ranks that really run, so the kernels of
    one rank of a larger job can be timed without its peers (the outputs are then partial sums only)."""
    import math

    if exchange not in ("peer", "nccl"):
        raise ValueError("exchange must be 'peer' or 'nccl'")
    ex = PeerExchange(rank=rank, world=world, max_rows=batch, d=shape.d) if exchange == "peer" else None
    if ex is not None and trace:
        ex.start_trace()
    part_rank, part_world = (0, int(shard_of)) if shard_of else (rank, world)

    L = shape.n_layers if n_layers is None else int(n_layers)
    d, HD, KD, I = shape.d, shape.H * shape.Dh, shape.Hk * shape.Dh, shape.I
    S_max = ctx + max_new + 4
    layers = []
    for li in range(L):
        gen = torch.Generator(device=device).manual_seed(seed * 100003 + li)

        def w(out_f, in_f):
            t = torch.randn(out_f, in_f, device=device, dtype=torch.float32, generator=gen)
            return (t / math.sqrt(in_f)).to(dtype)

        full = {"q_v": w(shape.Rq, d), "q_u": w(HD, shape.Rq), "k_v": w(shape.Rk, d), "k_u": w(KD, shape.Rk),
                "v_v": w(shape.Rv, d), "v_u": w(KD, shape.Rv), "o_v": w(shape.Ro, HD), "o_u": w(d, shape.Ro),
                "gate_v": w(shape.Rg, d), "gate_u": w(I, shape.Rg), "up_v": w(shape.Ru, d), "up_u": w(I, shape.Ru),
                "down_v": w(shape.Rd, I), "down_u": w(d, shape.Rd),
                "ln1": torch.ones(d, device=device, dtype=dtype), "ln2": torch.ones(d, device=device, dtype=dtype)}
        sh = shard_layer_weights(full, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=part_rank, world=part_world)
        layer = TPDecodeLayer(sh, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=part_rank, world=part_world, batch=batch,
                              S_max=S_max, eps=shape.eps, device=device, dtype=dtype, exchange=ex)
        if ctx > 0:
            g2 = torch.Generator(device=device).manual_seed(seed * 100003 + 7919 + li * world + rank)
            layer.k_cache[:, :ctx].copy_(torch.randn(layer.k_cache[:, :ctx].shape, device=device, generator=g2).to(dtype))
            layer.v_cache[:, :ctx].copy_(torch.randn(layer.v_cache[:, :ctx].shape, device=device, generator=g2).to(dtype))
        layers.append(layer)
        del full, sh
    gen = torch.Generator(device=device).manual_seed(seed * 100003 + 999983)
    embed = (torch.randn(shape.vocab, d, device=device, dtype=torch.float32, generator=gen) / math.sqrt(d)).to(dtype)
    lm_head = (torch.randn(shape.vocab, d, device=device, dtype=torch.float32, generator=gen) / math.sqrt(d)).to(dtype)
    model = TPModel(layers, embed, torch.ones(d, device=device, dtype=dtype), lm_head, batch=batch, S_max=S_max,
                    head_dim=shape.Dh, theta=shape.theta, eps=shape.eps, device=device, dtype=dtype, use_graph=use_graph)
    model.exchange = ex
    model.seqlens.fill_(ctx)
    model.tokens.copy_(torch.arange(batch, device=device) % shape.vocab)
    return model
