"""A Llama-2-7B-shaped mixed-precision decode stack made only of the packed linears, optionally split
column-parallel on N over the GPUs of one node.

This is the multi-GPU form of the packed linear path; the reference is single-GPU and has no
counterpart.  Per transformer block the four decode launches are
    fused QKV   [3*d/g rows  <- d]      (one launch, three outputs: the rank's Q, K and V heads)
    o_proj      [d/g rows    <- d]
    gate/up     [2*f/g rows  <- d]      (the fused silu(gate)*up kernel, f/g outputs)
    down        [d/g rows    <- f]
with d = 4096, f = 11008, every block at its own bit-width from {2, 3, 4}.  Every rank holds the
rows [r*n/g, (r+1)*n/g) of each matrix (Q, K, V by whole heads; gate and up by the same rows) and
the full activation; after each launch the [B, n/g] slice that the next launch consumes is
all-gathered over NVLink, so that every rank again holds the full [B, n] activation (four gathers per
block: Q, o_proj, gate/up, down; the K and V slices stay on their rank, as their consumer --
attention -- is head-parallel).  Two gather implementations: `comm="nccl"` calls NCCL's all-gather after
each launch; `comm="p2p"` fuses the gather into the decode kernel -- every output element is stored
straight into all ranks' peer-mapped activation buffers, and the kernel itself waits for its peers before
it reads its activations and publishes its completion to them, so a block is four launches and nothing
else; `comm="p2p_barrier"` keeps the stores but separates the hand-shake into a one-CTA barrier kernel
after each launch; `comm="p2p_seq"` numbers the launches of a step: a launch waits in the kernel for the flags of its
predecessor on every rank (not for a completion event on its own GPU), and a one-CTA kernel after each launch
publishes its completion; a block's QKV launch, which reads x and not the previous block's output, waits for one
launch less and so overlaps the previous hand-shake.

Only the linears and the gathers are in the step: attention, normalisation and residual adds of a
real model are other kernels and are outside this path.  Each block reads the step's hidden state
x; inside a block the data flows  x -> QKV -> (Q part) -> o_proj -> gate/up -> down.

The synthetic weights are drawn on the stack's device (seeded per block and matrix, identical on every
rank) and quantised and packed by `packer`: by default the library's GPU kernel (cb_quantize_pack, which is
bit-identical to the reference's CPU packer); the CPU tests of the sharding arithmetic pass one built on
their oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .ops import PackedLinearWeight, fused_gate_up, fused_qkv, new_workspace, packed_linear

LLAMA2_7B = dict(n_blocks=32, d_model=4096, d_ff=11008)


def sample_bitmap(n_blocks: int = 32, seed: int = 0) -> List[int]:
    """Seeded uniform draw of a per-block bit-width from {2, 3, 4}, the draw of the reference's
    Crispybits/quantization/scripts/sample_bitmaps.py:11-12 (seed 0 gives mean 3.06 bits over 32 blocks)."""
    rng = np.random.default_rng(seed)
    return [int(b) for b in rng.choice(np.array([2, 3, 4], dtype=np.int8), size=n_blocks, replace=True)]


# ------------------------------------------------------------------ quantise + pack
def gpu_packer(w: torch.Tensor, bits: int, group_size: int = 128, dtype=torch.float16) -> PackedLinearWeight:
    """Quantise and pack a float32 [N, K] CUDA matrix with the library's kernel (cb_quantize_pack, bit-identical to
    the reference's CPU packer)."""
    from . import _C
    packed, scales, zeros = _C.quantize_pack(w, bits, group_size, dtype)
    return PackedLinearWeight(packed, scales, zeros, bits, group_size, w.shape[1], w.shape[0])


def _rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0]
    assert n % world == 0
    return w[rank * n // world:(rank + 1) * n // world]


@dataclass
class _Block:
    bits: int
    qkv: PackedLinearWeight
    q: PackedLinearWeight
    k: PackedLinearWeight
    v: PackedLinearWeight
    o: PackedLinearWeight
    gate: PackedLinearWeight
    up: PackedLinearWeight
    down: PackedLinearWeight


class DecodeStack:
    """The packed linears of `n_blocks` transformer blocks on one rank of a `world`-way column split."""

    def __init__(self, n_blocks: int = 32, d_model: int = 4096, d_ff: int = 11008, bitmap: Optional[List[int]] = None,
                 rank: int = 0, world: int = 1, device="cuda", seed: int = 0, std: float = 0.02, group_size: int = 128,
                 comm: str = "nccl", packer=None):
        quantize_pack = packer if packer is not None else gpu_packer
        if d_model % world or d_ff % world or (d_model // world) % 2:
            raise ValueError("d_model and d_ff must divide evenly over the ranks")
        self.n_blocks, self.d_model, self.d_ff = n_blocks, d_model, d_ff
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.bitmap = list(bitmap) if bitmap is not None else sample_bitmap(n_blocks, seed)
        if len(self.bitmap) != n_blocks:
            raise ValueError("bitmap length does not match the number of blocks")
        if comm not in ("nccl", "p2p", "p2p_barrier", "p2p_seq"):
            raise ValueError(comm)
        self.comm = comm if world > 1 else "nccl"
        self.blocks: List[_Block] = []
        self.workspace = new_workspace(self.device)
        gen = torch.Generator(device=self.device)

        def draw(block: int, which: int, n: int, k: int) -> torch.Tensor:
            gen.manual_seed(1_000_003 * seed + 97 * block + which)       # same full matrix on every rank
            return torch.randn(n, k, generator=gen, device=self.device, dtype=torch.float32) * std

        for i, bits in enumerate(self.bitmap):
            # this rank's Q, K, V heads live in one row-concatenated matrix; q / k / v are row slices of it
            qkv = quantize_pack(torch.cat([_rows(draw(i, j, d_model, d_model), rank, world) for j in (1, 2, 3)]), bits, group_size)
            dl = d_model // world

            def part(j, w=qkv, dl=dl):
                return PackedLinearWeight(w.packed[j * dl:(j + 1) * dl], w.scales[j * dl:(j + 1) * dl],
                                          w.zeros[j * dl:(j + 1) * dl], w.bits, w.group_size, w.in_features, dl)

            blk = _Block(
                bits=bits, qkv=qkv, q=part(0), k=part(1), v=part(2),
                o=quantize_pack(_rows(draw(i, 4, d_model, d_model), rank, world), bits, group_size),
                gate=quantize_pack(_rows(draw(i, 5, d_ff, d_model), rank, world), bits, group_size),
                up=quantize_pack(_rows(draw(i, 6, d_ff, d_model), rank, world), bits, group_size),
                down=quantize_pack(_rows(draw(i, 7, d_model, d_ff), rank, world), bits, group_size))
            self.blocks.append(blk)

    # -------------------------------------------------------------- sizes
    def algorithmic_bytes(self, batch: int) -> int:
        """Bytes one rank must move per step: packed words + fp16 scales and zeros of its shards, plus the
        activations read and written by its launches (weights counted once for any batch <= 8)."""
        total = 0
        for blk in self.blocks:
            for w in (blk.qkv, blk.o, blk.gate, blk.up, blk.down):
                total += w.packed.numel() * 4 + w.scales.numel() * 2 * 2
            total += batch * 2 * (self.d_model + 3 * blk.q.out_features)         # QKV in / out
            total += batch * 2 * (self.d_model + blk.o.out_features)
            total += batch * 2 * (self.d_model + blk.gate.out_features)
            total += batch * 2 * (self.d_ff + blk.down.out_features)
        return total

    def launches_per_step(self) -> int:
        return (8 if self.comm in ("p2p_barrier", "p2p_seq") else 4) * self.n_blocks   # own kernels; NCCL's are not counted

    # -------------------------------------------------------------- peer-mapped buffers for comm="p2p"
    def _setup_p2p(self, max_batch: int = 8):
        """One symmetric allocation per rank: gathered activations Q, A (o_proj out), Y (down out) [8, d], M
        (gate/up out) [8, f], then the barrier flags.  Every rank learns every peer's base address."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        d, f, esz = self.d_model, self.d_ff, 2
        self._off = {"q": 0, "a": max_batch * d * esz, "y": 2 * max_batch * d * esz, "m": 3 * max_batch * d * esz}
        self._off["flags"] = (3 * max_batch * d * esz + max_batch * f * esz + 255) // 256 * 256
        total = self._off["flags"] + 256
        self._symm = symm.empty(total, dtype=torch.uint8, device=self.device)
        self._symm.zero_()
        self._hdl = symm.rendezvous(self._symm, dist.group.WORLD)
        self._peer_base = [int(p) for p in self._hdl.buffer_ptrs]
        self._epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._pstatus = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._done = torch.zeros(1, dtype=torch.int32, device=self.device)
        from . import _C
        flags = [b + self._off["flags"] for b in self._peer_base]
        self._sync = _C.PeerSync(flags, self._symm[self._off["flags"]:self._off["flags"] + 256], self._epoch,
                                 self._done, self._pstatus, self.rank, numbered=self.comm == "p2p_seq") \
            if self.comm in ("p2p", "p2p_seq") else None
        self._local = {k: self._symm[o:] for k, o in self._off.items()}
        self._qkv_local = None
        torch.cuda.synchronize()
        dist.barrier()

    def _buf(self, name: str, batch: int, width: int) -> torch.Tensor:
        return self._local[name][: batch * width * 2].view(torch.float16).view(batch, width)

    def _barrier(self):
        if self._sync is not None and self._sync.numbered:
            from . import _C
            _C.peer_publish(self._sync, self._seq)      # launch `seq` of the step is complete on this rank
            self._seq += 1
            return
        if self._sync is not None:
            return          # the decode kernels carry the hand-shake
        from . import _C
        _C.peer_barrier([b + self._off["flags"] for b in self._peer_base], self._local["flags"][:256], self._epoch,
                        self._pstatus, self.rank)

    def _step_p2p(self, x: torch.Tensor) -> torch.Tensor:
        from . import _C
        from .ops import _resolve
        if not hasattr(self, "_symm"):
            self._setup_p2p()
        B, d, f, g, r = x.shape[0], self.d_model, self.d_ff, self.world, self.rank
        dl, fl = d // g, f // g
        peers = lambda name: [b + self._off[name] for b in self._peer_base]
        if self._qkv_local is None or self._qkv_local.shape[0] != B:
            self._qkv_local = torch.empty(B, 3 * dl, dtype=torch.float16, device=self.device)
            self._o_local = torch.empty(B, dl, dtype=torch.float16, device=self.device)
            self._m_local = torch.empty(B, fl, dtype=torch.float16, device=self.device)
        none = torch.empty(0, dtype=torch.float16, device=self.device)
        sk = lambda rows, k: _resolve(None, 1, B, rows, k, self.device, torch.float16, self.blocks[0].o.group_size)
        xq, xa, xm, xy = self._buf("q", B, d), self._buf("a", B, d), self._buf("m", B, f), self._buf("y", B, d)
        self._seq = 0                    # numbered hand-shake: launches of the step in issue order
        for blk in self.blocks:
            w = blk.qkv
            # QKV reads the step's input, not what the previous launch gathered: it only has to know that nobody still
            # reads the Q buffer it overwrites (the previous block's o_proj, three launches back), which the launch
            # before it has already waited for -- so it asks for one launch less and overlaps that launch's hand-shake
            _C.packed_gemv_scatter(x, w.packed, w.scales, w.zeros, none, self._qkv_local, peers("q"), dl, d, r * dl,
                                   w.bits, d, w.group_size, sk(3 * dl, d), 1, 0, self._sync, self._seq,
                                   max(0, self._seq - 1))
            self._barrier()
            w = blk.o
            _C.packed_gemv_scatter(xq, w.packed, w.scales, w.zeros, none, self._o_local, peers("a"), dl, d, r * dl,
                                   w.bits, d, w.group_size, sk(dl, d), 1, 0, self._sync, self._seq)
            self._barrier()
            wg, wu = blk.gate, blk.up
            _C.fused_gate_up_scatter(xa, wg.packed, wg.scales, wg.zeros, wu.packed, wu.scales, wu.zeros, self._m_local,
                                     peers("m"), fl, f, r * fl, wg.bits, d, wg.group_size, sk(2 * fl, d), 1, self._sync,
                                     self._seq)
            self._barrier()
            w = blk.down
            _C.packed_gemv_scatter(xm, w.packed, w.scales, w.zeros, none, self._o_local, peers("y"), dl, d, r * dl,
                                   w.bits, f, w.group_size, sk(dl, f), 1, 0, self._sync, self._seq)
            self._barrier()
        if self._sync is not None and self._sync.numbered:
            _C.peer_step_end(self._sync, self._seq)     # every rank has published the whole step; the base moves on
        elif self._sync is not None:
            _C.peer_wait(self._sync)     # the peers' last slices have landed before anyone reads the result
        return xy

    def peer_status(self) -> int:
        """0 when every barrier heard from every peer in time (after a synchronize)."""
        return int(self._pstatus.item()) if hasattr(self, "_pstatus") else 0

    # -------------------------------------------------------------- one decode step
    def gather(self, t: torch.Tensor) -> torch.Tensor:
        """[B, n/g] on every rank -> [B, n] on every rank.  NCCL all-gather over NVLink; the batch > 1 case
        needs one transpose because the collective concatenates rank-major."""
        if self.world == 1:
            return t
        import torch.distributed as dist
        b, nl = t.shape
        out = torch.empty(self.world * b, nl, dtype=t.dtype, device=t.device)      # rank-major rows
        dist.all_gather_into_tensor(out, t.contiguous())
        if b == 1:
            return out.view(1, self.world * nl)
        return out.view(self.world, b, nl).permute(1, 0, 2).reshape(b, self.world * nl)

    def step(self, x: torch.Tensor, decode_threshold: int = 8) -> torch.Tensor:
        """x [B, d_model] (replicated on every rank) -> the last block's down-projection output [B, d_model]."""
        if self.comm != "nccl":
            return self._step_p2p(x)
        y = None
        kw = dict(decode_threshold=decode_threshold, workspace=self.workspace)
        for blk in self.blocks:
            oq, _ok, _ov = fused_qkv(x, blk.q, blk.k, blk.v, **kw)
            a = self.gather(packed_linear(self.gather(oq), blk.o, **kw))
            m = self.gather(fused_gate_up(a, blk.gate, blk.up, **kw))
            y = self.gather(packed_linear(m, blk.down, **kw))
        return y                                          # the last block's output; every block ran the same launches

    # -------------------------------------------------------------- check value (fp32, any device)
    @torch.no_grad()
    def reference_step(self, x: torch.Tensor, full_blocks: "List[Dict[str, torch.Tensor]]") -> torch.Tensor:
        """fp32 evaluation of the same data flow from full (un-sharded) dequantised weights
        {"q","k","v","o","gate","up","down"} per block; used by the tests."""
        y = None
        xf = x.float()
        for wd in full_blocks:
            q = xf @ wd["q"].T
            a = (q.half().float()) @ wd["o"].T
            a16 = a.half().float()
            m = torch.nn.functional.silu(a16 @ wd["gate"].T) * (a16 @ wd["up"].T)
            y = m.half().float() @ wd["down"].T
        return y
