"""Quantised linear layers over the decode-matmul operator, and the Llama-style stack of them.

``DecodeLinear`` holds one weight matrix as tile-packed codes plus codebook and scale.
``LinearStack`` chains the four projections of a transformer block (qkv, o, gate+up, down)
for a number of layers and shards them over the ranks of a tensor-parallel group:
qkv and gate/up are column-parallel (split N: a contiguous byte range of the tiled codes),
o and down are row-parallel (split K: tile-packed per shard) followed by an all-reduce.
"""
from __future__ import annotations

import torch

from . import _lib, ops
from .layout import shard_cols, shard_fused_rows, transpose_tile


class DecodeLinear:
    """y = scale * x @ W^T with W stored as 2-bit-per-weight codes (fp16 family).

    ``codes`` is the LOGICAL int16 [N, K/8] matrix; it is tile-packed here, once."""

    def __init__(self, codes: torch.Tensor, codebook_fp16: torch.Tensor, scale: float = 1.0, *, tiled: bool = False):
        self.codes = codes.contiguous() if tiled else transpose_tile(codes)
        self.codebook = codebook_fp16.contiguous()
        self.scale = float(scale)
        self.out_features = self.codes.shape[0]
        self.in_features = self.codes.shape[1] * 8

    @property
    def code_bytes(self) -> int:
        return self.codes.numel() * 2

    def to(self, device):
        self.codes = self.codes.to(device)
        self.codebook = self.codebook.to(device)
        return self

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
                 path: int = _lib.PATH_AUTO, pdl: bool = True) -> torch.Tensor:
        return ops.decode_matmul_fp16(x, self.codes, self.codebook, self.scale, out, path=path,
                                      accumulate=accumulate, pdl=pdl)


def llama_shapes(hidden: int, kv_heads: int, head_dim: int, ffn: int) -> dict:
    """(N, K) of the four fused projections of one block."""
    return {
        "qkv": (hidden + 2 * kv_heads * head_dim, hidden),
        "o": (hidden, hidden),
        "gate_up": (2 * ffn, hidden),
        "down": (hidden, ffn),
    }


LLAMA2_70B = dict(hidden=8192, kv_heads=8, head_dim=128, ffn=28672, layers=80)
LLAMA2_7B = dict(hidden=4096, kv_heads=32, head_dim=128, ffn=11008, layers=32)


class LinearStack:
    """The linear layers of ``layers`` transformer blocks with synthetic (seeded) codes.

    Data flow of one step for a [B, hidden] fp32 residual stream h:
        a = qkv(fp16(h));  h += o(fp16(a[:, :hidden]))          (attention itself is not part of
        g = gate_up(fp16(h));  h += down(fp16(silu(g0) * g1))    the operator: q stands in for it)
    Row-parallel outputs are summed over the tensor-parallel group before the residual add.
    By default the weights are generated directly in sharded form: rank r of w draws its own codes,
    so that no rank ever materialises a full matrix (what the benchmark needs at 17 GB).  With
    ``logical_seed`` every rank instead draws the same LOGICAL matrices from one seed and keeps its
    shard of them (q, k, v and gate, up sharded part by part, o and down by reduction index, each
    shard tile-packed on its own): the result then does not depend on the number of ranks, which is
    what the tensor-parallel tests compare.  Meant for small configurations."""

    def __init__(self, cfg: dict, codebook_fp16: torch.Tensor, device, world: int = 1, rank: int = 0,
                 seed: int = 46, scale: float = 2.0 ** -7, group=None, logical_seed: int | None = None,
                 tp_mode: str | None = None):
        self.cfg, self.world, self.rank, self.group = cfg, world, rank, group
        self.tp_mode = tp_mode  # None: by rank count and DMM_TP_MODE; "slots" | "pull" | "push" | "nccl"
        self.device = torch.device(device)
        self.hidden, self.ffn = cfg["hidden"], cfg["ffn"]
        shapes = llama_shapes(cfg["hidden"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"])
        for name, (n, k) in shapes.items():
            div = n if name in ("qkv", "gate_up") else k
            if div % (32 * world) or (name in ("qkv", "gate_up") and n % (16 * world)):
                raise RuntimeError(f"{name} does not shard over {world} ranks")
        if (cfg["kv_heads"] * cfg["head_dim"]) % (16 * world) or cfg["hidden"] % (32 * world) or cfg["ffn"] % (32 * world):
            raise RuntimeError(f"q/k/v or gate/up do not shard part by part over {world} ranks")
        self.shapes = shapes
        cb = codebook_fp16.to(self.device)
        gen = torch.Generator(device=self.device).manual_seed(
            logical_seed if logical_seed is not None else seed * 1000 + rank)
        kv = cfg["kv_heads"] * cfg["head_dim"]
        fused_parts = {"qkv": (cfg["hidden"], kv, kv), "gate_up": (cfg["ffn"], cfg["ffn"])}
        self.layers = []
        self.code_bytes_local = 0
        for _ in range(cfg["layers"]):
            block = {}
            for name, (n, k) in shapes.items():
                if name in ("qkv", "gate_up"):
                    n_loc, k_loc = n // world, k
                else:
                    n_loc, k_loc = n, k // world
                if logical_seed is not None:
                    logical = torch.randint(-32768, 32768, (n, k // 8), dtype=torch.int16, device=self.device,
                                            generator=gen)
                    if name in fused_parts:
                        mine = shard_fused_rows(logical, fused_parts[name], world, rank)
                    else:
                        mine = shard_cols(logical, world, rank)
                    block[name] = DecodeLinear(mine.contiguous(), cb, scale)
                else:
                    # uniform int16 codes; any bit pattern is a valid tile-packed matrix, so the
                    # shard is drawn directly in tiled form
                    codes = torch.randint(-32768, 32768, (n_loc, k_loc // 8), dtype=torch.int16, device=self.device,
                                          generator=gen)
                    block[name] = DecodeLinear(codes, cb, scale, tiled=True)
                self.code_bytes_local += block[name].code_bytes
            self.layers.append(block)
        self.code_bytes_total = sum(n * k // 4 for n, k in shapes.values()) * cfg["layers"]
        self.launches_per_step = 4 * cfg["layers"]
        # blocks per chained launch of the fused step; 0 = one launch per product, which measured
        # faster on B200 (77.5 against 91 us per block): the hardware's dependent-launch hand-over
        # beats a software barrier between resident CTAs
        self.chain_blocks = 0

    def step(self, h: torch.Tensor, path: int = _lib.PATH_AUTO, fused: bool | None = None) -> torch.Tensor:
        """One pass of the stack over the fp32 residual stream ``h`` [B, hidden] (updated in place).

        ``fused`` (default: whenever the batch is at most 32): every elementwise step between two
        layers runs inside the matmul kernels -- the loaders read fp32 and round to fp16 or form
        silu(gate) * up, the epilogues add onto the residual stream with atomic adds, and each
        kernel clears the buffer a later kernel accumulates into.  Four launches per block."""
        if fused is None:
            fused = h.shape[0] <= 32 and path == _lib.PATH_AUTO
        if fused:
            return self._step_fused(h)
        hid_loc = self.hidden // self.world
        ffn_loc = self.ffn // self.world
        for blk in self.layers:
            a = blk["qkv"](h.to(torch.float16), path=path)
            # row-parallel o: this rank's slice of the attention output stands in for attention
            a16 = a[:, :hid_loc].to(torch.float16).contiguous()
            self._row_parallel(blk["o"], a16, h, path)
            g = blk["gate_up"](h.to(torch.float16), path=path)
            act = (torch.nn.functional.silu(g[:, :ffn_loc]) * g[:, ffn_loc:]).to(torch.float16)
            self._row_parallel(blk["down"], act, h, path)
        return h

    def _buffers(self, batch: int):
        key = (batch,)
        if getattr(self, "_buf_key", None) != key:
            n_qkv = self.layers[0]["qkv"].out_features
            n_gu = self.layers[0]["gate_up"].out_features
            mk = lambda n: torch.zeros((batch, n), dtype=torch.float32, device=self.device)
            self._buf = {"a": mk(n_qkv), "g": mk(n_gu), "po": mk(self.hidden), "pd": mk(self.hidden)}
            # scratch of this stack's own (two stacks on two streams must not share the library's buffer)
            from .ops import workspace_bytes

            need = max(workspace_bytes(batch, lin.out_features, lin.in_features) for lin in self.layers[0].values())
            self._buf["ws"] = torch.zeros((need,), dtype=torch.uint8, device=self.device)
            self._buf_key = key
        return self._buf

    def _peer_state(self, batch: int):
        """Symmetric (peer-mapped) buffers for the tensor-parallel step: two copies of the residual
        stream and the flag words of the rank barrier.  None when symmetric memory cannot be set
        up (or DMM_TP_PEER=0): the step then sums with NCCL all-reduce."""
        import os

        key = (batch,)
        if getattr(self, "_peer_key", None) == key:
            return self._peer
        self._peer_key, self._peer = key, None
        if self.world == 1 and self.tp_mode == "slots":
            # a group of one: the same kernels on ordinary local buffers (what the one-GPU tests run)
            slots = torch.zeros((2, 1, batch, self.hidden), dtype=torch.float32, device=self.device)
            sflags = torch.zeros((64,), dtype=torch.int32, device=self.device)
            self._peer = dict(slots=slots, sflags=sflags, slot_ptrs=[slots.data_ptr()], sflag_ptrs=[sflags.data_ptr()],
                              h2=torch.zeros((2, batch, self.hidden), dtype=torch.float32, device=self.device))
            return self._peer
        if self.world == 1 or os.environ.get("DMM_TP_PEER", "1") == "0" or self.tp_mode == "nccl":
            return None
        # the kernels use plain peer loads and stores only: keep the buffers off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        ok = torch.zeros(1, device=self.device)
        try:
            import torch.distributed._symmetric_memory as symm

            group = self.group if self.group is not None else torch.distributed.group.WORLD
            res = symm.empty((2, batch, self.hidden), dtype=torch.float32, device=self.device)
            flags = symm.empty((64,), dtype=torch.int32, device=self.device)
            slots = symm.empty((2, self.world, batch, self.hidden), dtype=torch.float32, device=self.device)
            sflags = symm.empty((64,), dtype=torch.int32, device=self.device)
            for t in (res, flags, slots, sflags):
                t.zero_()
            h_res, h_flags = symm.rendezvous(res, group), symm.rendezvous(flags, group)
            h_slots, h_sflags = symm.rendezvous(slots, group), symm.rendezvous(sflags, group)
            nbytes = batch * self.hidden * 4
            peer = dict(res=res, flags=flags, cur=0, mode=os.environ.get("DMM_TP_MODE", "pull"),
                        res_ptrs=[[int(ptr) + i * nbytes for ptr in h_res.buffer_ptrs] for i in range(2)],
                        flag_ptrs=[int(ptr) for ptr in h_flags.buffer_ptrs],
                        slots=slots, sflags=sflags, slot_ptrs=[int(ptr) for ptr in h_slots.buffer_ptrs],
                        sflag_ptrs=[int(ptr) for ptr in h_sflags.buffer_ptrs],
                        h2=torch.zeros((2, batch, self.hidden), dtype=torch.float32, device=self.device))
            ok.fill_(1)
        except Exception:  # no peer mapping on this system: every rank must fall back together
            peer = None
        torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN, group=self.group)
        torch.cuda.synchronize(self.device)
        self._peer = peer if float(ok.item()) == 1.0 else None
        return self._peer

    def _step_fused_peer(self, h: torch.Tensor, peer) -> torch.Tensor:
        """Tensor-parallel fused step without collectives: the row-parallel kernels add their
        partial products into the residual buffer of EVERY rank through peer memory, and a
        barrier kernel orders the ranks.  The residual stream alternates between two buffers, so a
        rank never adds into a buffer that a slower rank still reads (the kernel that adds first
        moves this rank's own copy over and leaves the old buffer zero)."""
        from .ops import decode_matmul_fused as mm
        from .ops import decode_matmul_fused_tp as mm_tp
        from .ops import xrank_barrier

        B = h.shape[0]
        buf = self._buffers(B)
        a, g = buf["a"], buf["g"]
        hid_loc, ffn_loc = self.hidden // self.world, self.ffn // self.world
        res, cur = peer["res"], peer["cur"]
        res[cur].copy_(h)  # the other buffer is zero (invariant kept by every row-parallel kernel)
        a.zero_()
        kw = dict(accumulate=True, atomic=True, pdl=True, workspace=buf["ws"])
        for blk in self.layers:
            q, o, gu, dn = blk["qkv"], blk["o"], blk["gate_up"], blk["down"]
            mm(res[cur], q.codes, q.codebook, q.scale, a, x_kind=_lib.X_F32, zero=g, **kw)
            mm_tp(a, o.codes, o.codebook, o.scale, peer["res_ptrs"][1 - cur], (B, self.hidden), x_kind=_lib.X_F32, pdl=True,
                  move_src=res[cur], move_dst=res[1 - cur])
            xrank_barrier(peer["flag_ptrs"], self.rank, self.device)
            cur = 1 - cur
            mm(res[cur], gu.codes, gu.codebook, gu.scale, g, x_kind=_lib.X_F32, zero=a, **kw)
            mm_tp(g, dn.codes, dn.codebook, dn.scale, peer["res_ptrs"][1 - cur], (B, self.hidden),
                  x_kind=_lib.X_F32_SILU_MUL, x_gap=ffn_loc, pdl=True, move_src=res[cur], move_dst=res[1 - cur])
            xrank_barrier(peer["flag_ptrs"], self.rank, self.device)
            cur = 1 - cur
        h.copy_(res[cur])
        res[cur].zero_()  # restores the starting state: both buffers zero, so `cur` may restart at 0
        return h

    def _step_fused_slots(self, h: torch.Tensor, peer) -> torch.Tensor:
        """Tensor-parallel fused step with compute and collective in the matmul kernels: a row-parallel
        kernel's last CTA copies the finished partial product into this rank's slot on every rank and
        raises a flag; the loaders of the column-parallel kernel that follows wait for all ranks' flags and
        read the residual stream plus all slots (writing the sum back as the new residual stream).  One
        NVLink traversal per row-parallel layer, no barrier, no reduction kernel; four launches per block
        as on one GPU.  The residual stream alternates between two local buffers."""
        from . import ops as _ops

        B = h.shape[0]
        buf = self._buffers(B)
        a, g = buf["a"], buf["g"]
        hid_loc, ffn_loc = self.hidden // self.world, self.ffn // self.world
        h2, slots, sflags = peer["h2"], peer["slots"], peer["sflags"]
        sp, fp, w, r = peer["slot_ptrs"], peer["sflag_ptrs"], self.world, self.rank
        cur = 0
        h2[cur].copy_(h)
        a.zero_()
        kw = dict(accumulate=True, atomic=True, pdl=True, workspace=buf["ws"])
        mm, hint = _ops.decode_matmul_fused, _ops.hint_next_weights
        for i, blk in enumerate(self.layers):
            q, o, gu, dn = blk["qkv"], blk["o"], blk["gate_up"], blk["down"]
            nxt = self.layers[i + 1]["qkv"].codes if i + 1 < len(self.layers) else None
            hint(o.codes)
            if i == 0:  # nothing pending from a row-parallel layer yet
                mm(h2[cur], q.codes, q.codebook, q.scale, a, x_kind=_lib.X_F32, zero=g, **kw)
            else:       # the partial products of the previous block's down projection arrive through the slots
                _ops.tp_consume(h2[cur], h2[1 - cur], slots, sflags, w, q.codes, q.codebook, q.scale, a, pdl=True, zero=g)
                cur = 1 - cur
            hint(gu.codes)
            _ops.tp_produce(a, o.codes, o.codebook, o.scale, sp, fp, r, self.hidden, x_kind=_lib.X_F32, pdl=True)
            hint(dn.codes)
            _ops.tp_consume(h2[cur], h2[1 - cur], slots, sflags, w, gu.codes, gu.codebook, gu.scale, g, pdl=True, zero=a)
            cur = 1 - cur
            hint(nxt)
            _ops.tp_produce(g, dn.codes, dn.codebook, dn.scale, sp, fp, r, self.hidden, x_kind=_lib.X_F32_SILU_MUL,
                            x_gap=ffn_loc, pdl=True)
        _ops.tp_finalize(h2[cur], h, slots, sflags, w)
        return h

    def _step_fused_pull(self, h: torch.Tensor, peer) -> torch.Tensor:
        """Tensor-parallel fused step with a one-shot all-reduce kernel: a row-parallel layer
        accumulates its partial product into this rank's own symmetric buffer, then one kernel waits
        for all ranks, pulls every rank's partial over NVLink and adds the sum to the local residual.
        Two partial buffers alternate; the all-reduce of one layer clears the buffer of the layer
        before (all ranks have finished reading it by then), so one barrier per layer is enough."""
        import os

        from .ops import decode_matmul_fused as mm
        from .ops import xrank_allreduce_add

        B = h.shape[0]
        buf = self._buffers(B)
        a, g = buf["a"], buf["g"]
        ffn_loc = self.ffn // self.world
        part, cur = peer["res"], peer["cur"]
        a.zero_()
        kw = dict(accumulate=True, atomic=True, pdl=True, workspace=buf["ws"])
        from . import ops as _ops

        hint = lambda w: _ops.hint_next_weights(w)
        for i, blk in enumerate(self.layers):
            q, o, gu, dn = blk["qkv"], blk["o"], blk["gate_up"], blk["down"]
            nxt = self.layers[i + 1]["qkv"].codes if i + 1 < len(self.layers) else None
            hint(o.codes)
            mm(h, q.codes, q.codebook, q.scale, a, x_kind=_lib.X_F32, zero=g, **kw)
            hint(gu.codes)
            mm(a, o.codes, o.codebook, o.scale, part[cur], x_kind=_lib.X_F32, **kw)
            xrank_allreduce_add(h, peer["res_ptrs"][cur], peer["flag_ptrs"], self.rank, zero=part[1 - cur])
            cur = 1 - cur
            hint(dn.codes)
            mm(h, gu.codes, gu.codebook, gu.scale, g, x_kind=_lib.X_F32, zero=a, **kw)
            hint(nxt)
            mm(g, dn.codes, dn.codebook, dn.scale, part[cur], x_kind=_lib.X_F32_SILU_MUL, x_gap=ffn_loc, **kw)
            xrank_allreduce_add(h, peer["res_ptrs"][cur], peer["flag_ptrs"], self.rank, zero=part[1 - cur])
            cur = 1 - cur
        peer["cur"] = cur  # an even number of row-parallel layers brings it back to where it started
        return h

    def _step_fused(self, h: torch.Tensor) -> torch.Tensor:
        from .ops import decode_matmul_fused as mm

        if (self.world > 1 or self.tp_mode == "slots") and h.shape[0] <= 32:
            import os

            peer = self._peer_state(h.shape[0])
            if peer is not None:
                # The slots form (no cross-rank kernel, no barrier) is the fastest at every rank count measured on
                # B200 at batch 1 (ms per step of the Llama-2-70B stack at 2 / 4 / 8 ranks: slots 5.11 / 4.03 / 3.81,
                # push 5.22 / 4.83 / 4.97, pull 5.16 / 5.06 / 5.97); it splits the activations inside the kernel, so larger batches take the
                # one-shot all-reduce kernel (few ranks) or the epilogues that add into every rank (many ranks).
                default = "slots" if h.shape[0] <= 8 else ("pull" if self.world <= 2 else "push")
                mode = self.tp_mode or os.environ.get("DMM_TP_MODE", default)
                if mode == "slots" and h.shape[0] > 8 and self.world > 2:
                    mode = "push"
                if mode == "slots" and h.shape[0] > 8:
                    mode = "pull"  # the slots form splits the activations inside the kernel: small batches only
                self.tp_form_used = mode  # what a step of this stack ran last: "slots" | "push" | "pull"
                if mode == "slots":
                    return self._step_fused_slots(h, peer)
                if mode == "push":
                    return self._step_fused_peer(h, peer)
                return self._step_fused_pull(h, peer)

        buf = self._buffers(h.shape[0])
        a, g, po, pd = buf["a"], buf["g"], buf["po"], buf["pd"]
        hid_loc, ffn_loc = self.hidden // self.world, self.ffn // self.world
        tp = self.world > 1
        # Every output is accumulated with atomic adds, so it has to be zero when its kernel
        # starts.  Each kernel clears one buffer that is idle while it runs (after it has seen the
        # previous kernel finish): qkv clears g, o clears pd, gate_up clears a, down clears po.
        a.zero_()
        if tp:
            po.zero_()
        if not tp and h.shape[0] < 4 and self.chain_blocks > 0:
            # Small batch on one GPU: whole blocks as chains of dependent products in one launch
            # each (the CTAs stay resident, the decoders run ahead across the layer boundaries).
            from .ops import decode_matmul_chain

            for b0 in range(0, len(self.layers), self.chain_blocks):
                ops = []
                for blk in self.layers[b0:b0 + self.chain_blocks]:
                    q, o, gu, dn = blk["qkv"], blk["o"], blk["gate_up"], blk["down"]
                    ops += [dict(x=h, weights_compressed=q.codes, scale=q.scale, output=a, zero=g),
                            dict(x=a, weights_compressed=o.codes, scale=o.scale, output=h),
                            dict(x=h, weights_compressed=gu.codes, scale=gu.scale, output=g, zero=a),
                            dict(x=g, weights_compressed=dn.codes, scale=dn.scale, output=h,
                                 x_kind=_lib.X_F32_SILU_MUL, x_gap=ffn_loc)]
                decode_matmul_chain(ops, self.layers[b0]["qkv"].codebook, pdl=True)
            return h
        from . import ops as _ops

        hint = lambda w: _ops.hint_next_weights(w)
        for i, blk in enumerate(self.layers):
            q, o, gu, dn = blk["qkv"], blk["o"], blk["gate_up"], blk["down"]
            nxt = self.layers[i + 1]["qkv"].codes if i + 1 < len(self.layers) else None
            kw = dict(accumulate=True, atomic=True, pdl=True, workspace=buf["ws"])
            # before every product: which weights the product after it will stream (its kernel prefetches
            # their first codes into L2, so the next launch does not start with a DRAM round trip)
            hint(o.codes)
            mm(h, q.codes, q.codebook, q.scale, a, x_kind=_lib.X_F32, zero=g, **kw)
            hint(gu.codes)
            if tp:
                mm(a, o.codes, o.codebook, o.scale, po, x_kind=_lib.X_F32, zero=pd, **kw)
                torch.distributed.all_reduce(po, group=self.group)
                h.add_(po)
            else:
                mm(a, o.codes, o.codebook, o.scale, h, x_kind=_lib.X_F32, **kw)
            hint(dn.codes)
            mm(h, gu.codes, gu.codebook, gu.scale, g, x_kind=_lib.X_F32, zero=a, **kw)
            hint(nxt)
            if tp:
                mm(g, dn.codes, dn.codebook, dn.scale, pd, x_kind=_lib.X_F32_SILU_MUL, x_gap=ffn_loc, zero=po, **kw)
                torch.distributed.all_reduce(pd, group=self.group)
                h.add_(pd)
            else:
                mm(g, dn.codes, dn.codebook, dn.scale, h, x_kind=_lib.X_F32_SILU_MUL, x_gap=ffn_loc, **kw)
        return h

    def _row_parallel(self, lin: DecodeLinear, x16: torch.Tensor, h: torch.Tensor, path: int) -> None:
        if self.world == 1:
            lin(x16, out=h, accumulate=True, path=path)
            return
        part = lin(x16, path=path)
        torch.distributed.all_reduce(part, group=self.group)
        h.add_(part)
