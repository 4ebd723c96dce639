"""Tensor-parallel exchange over peer-mapped memory: the buffers, counters and call descriptors behind the fused
reduce-scatter / all-gather kernels (csrc/tp.cu, MFX_EPI_PEER_SCATTER in csrc/qmm_t.cu).

No counterpart in the single-device reference; it serves the column- / row-split QuantizedLinear layers of the
Qwen-Image blocks (src/mflux/models/qwen/model/qwen_transformer/qwen_transformer_block.py:27-76) when one image is
spread over the GPUs of a node. PyTorch supplies the plumbing only: `torch.distributed._symmetric_memory` allocates
one buffer per rank and maps every rank's buffer into every process; all traffic is this library's own kernels
storing to those mappings (plain stores over NVLink, no multicast, no TMA on peer memory).

Layout. Every rank owns R = ceil(S / world) consecutive rows of each sample's joint sequence (text rows first).
The symmetric buffer of a rank holds
    nbuf   bf16 [batch, world * R, D]   the normalised activations of the WHOLE sequence: every rank writes its
                                         own rows into every rank's copy (all-gather by stores)
    part   bf16 [world, batch, R, D]    partial sums of a row-split linear for the rows this rank owns: rank j's
                                         matmul epilogue writes slot j (reduce-scatter by stores)
    flags  int32 [2 * world]            arrival counters: [0:world] one per source rank for `part`,
                                         [world:2*world] one per source rank for `nbuf`
Counters only grow; a consumer waits for ">= epoch". The epochs of a forward pass are offsets from a device-side
base that advances after every pass, so a pass recorded as a CUDA graph can be replayed.
"""
from __future__ import annotations

import torch

from . import _lib, ops

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


class PeerExchange:
    def __init__(self, group, rank: int, world: int, batch: int, seq: int, split: int, dim: int, device,
                 copy_engine_gather: bool = True):
        import torch.distributed._symmetric_memory as symm

        if world > _lib.TP_MAX_WORLD:
            raise ValueError(f"at most {_lib.TP_MAX_WORLD} tensor-parallel ranks")
        self.group, self.rank, self.world = group, rank, world
        self.batch, self.seq, self.split, self.dim = batch, seq, split, dim
        self.rows = -(-seq // world)               # R
        self.seq_pad = self.rows * world
        n_nbuf = batch * self.seq_pad * dim * 2
        n_part = world * batch * self.rows * dim * 2
        self._off_part = (n_nbuf + 255) // 256 * 256
        self._off_flags = self._off_part + (n_part + 255) // 256 * 256
        total = self._off_flags + 256
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group if group is not None else torch.distributed.group.WORLD)
        self.bases = [int(self.handle.buffer_ptrs[r]) for r in range(world)]
        self.nbuf = self.buf[:n_nbuf].view(torch.bfloat16).view(batch, self.seq_pad, dim)
        self.part = self.buf[self._off_part:self._off_part + n_part].view(torch.bfloat16).view(
            world, batch, self.rows, dim)
        self.flags = self.buf[self._off_flags:self._off_flags + 8 * world].view(torch.int32)
        self.local = torch.zeros(4, dtype=torch.int32, device=device)   # completion counts: [0] scatter, [1] fuse,
        # [2] scatter launches of a second stream (two scatters in flight at once must not share a count)
        self.epoch_base = torch.zeros(2, dtype=torch.int32, device=device)   # [0] part arrivals, [1] nbuf arrivals
        self.x = torch.zeros(batch, self.rows, dim, dtype=torch.float32, device=device)   # owned residual rows
        self.rs_count = self.ag_count = 0       # arrivals issued so far in the current forward pass
        # All-gather by the copy engines: tp_fuse stores the normalised rows locally only; this rank's rows then go
        # to every peer as stream-ordered device-to-device copies on a side stream (NVLink, no SMs), followed by
        # the arrival signal, while the main stream already runs the matmuls over the rank's own rows.
        self.copy_engine_gather = copy_engine_gather
        self.copy_stream = torch.cuda.Stream(device=device)
        self.peer_nbuf = [self.handle.get_buffer(r, (batch, self.seq_pad, dim), torch.bfloat16, 0)
                          for r in range(world)]
        self.ag_flag_ptrs = [self.bases[r] + self._off_flags + 4 * (world + rank) for r in range(world)]
        torch.cuda.synchronize(device)
        self.handle.barrier()                    # every rank's buffer is zeroed before anyone writes into it

    # row range of the joint sequence this rank owns
    @property
    def lo(self) -> int:
        return self.rank * self.rows

    @property
    def hi(self) -> int:
        return min(self.seq, (self.rank + 1) * self.rows)

    def begin(self) -> None:
        self.rs_count = self.ag_count = 0

    def end(self) -> None:
        """Advances the device-side epoch bases by what this pass added (stream-ordered, so capturable)."""
        if self.copy_engine_gather:
            self.join()
        self.epoch_base += self._delta()

    def _delta(self):
        """(part arrivals, nbuf arrivals) of this pass as a device tensor, made once per distinct pair."""
        key = (self.rs_count, self.ag_count)
        cache = self.__dict__.setdefault("_deltas", {})
        if key not in cache:
            cache[key] = torch.tensor(key, dtype=torch.int32, device=self.epoch_base.device)
        return cache[key]

    def scatter(self, row_offset: int, lane: int = 0) -> "_lib.TpScatter":
        """Descriptor for a row-split linear whose activation rows start at joint row `row_offset`. Launches that
        may run at the same time (different streams) take different `lane`s (0 or 1): each counts its own CTAs."""
        sc = _lib.TpScatter()
        sc.world, sc.rank, sc.rows_per_rank, sc.row_offset, sc.D = self.world, self.rank, self.rows, row_offset, self.dim
        for r in range(self.world):
            sc.dst[r] = self.bases[r] + self._off_part
            sc.flags[r] = self.bases[r] + self._off_flags + 4 * self.rank
        sc.done_counter = self.local.data_ptr() + (8 if lane else 0)
        self.rs_count += 1
        return sc

    def fuse(self, *, reduce: bool, bias=(None, None), gate=(None, None), shift=(None, None), scale=(None, None),
             eps: float = 1e-6) -> None:
        """tp_fuse on the owned rows. `bias`, `gate`, `shift`, `scale` are (text-segment, image-segment) pairs;
        gate / shift / scale are [batch, D] views of the modulation tensors (one dtype, one batch stride)."""
        a = _lib.TpFuseArgs()
        a.world, a.rank, a.batch, a.rows_per_rank = self.world, self.rank, self.batch, self.rows
        a.seq_pad, a.seq, a.split, a.D = self.seq_pad, self.seq, self.split, self.dim
        a.x = self.x.data_ptr()
        if reduce:
            a.partials = self.part.data_ptr()
            a.rs_flags = self.flags.data_ptr()
            a.rs_target = self.rs_count
            a.epoch_base = self.epoch_base.data_ptr()
        mods = [t for t in (*gate, *shift, *scale) if t is not None]
        if mods:
            a.mod_dtype = _DT[mods[0].dtype]
            strides = {t.stride(0) for t in mods}
            if len(strides) != 1 or any(t.dtype != mods[0].dtype or t.stride(-1) != 1 for t in mods):
                raise ValueError("gate, shift and scale must be [batch, D] views of one dtype and batch stride")
            a.mod_batch_stride = strides.pop()
        else:
            a.mod_dtype = _lib.BF16
        keep = []
        for s in range(2):
            if bias[s] is not None:
                b = bias[s].contiguous()
                keep.append(b)
                a.bias[s], a.bias_dtype = b.data_ptr(), _DT[b.dtype]
            for name, src in (("gate", gate), ("shift", shift), ("scale", scale)):
                if src[s] is not None:
                    getattr(a, name)[s] = src[s].data_ptr()
        a.eps = eps
        pushes = scale[0] is not None
        if pushes:
            for r in range(self.world):
                a.push_dst[r] = self.bases[r]
                a.ag_flags[r] = self.ag_flag_ptrs[r]
            a.push_local_only = int(self.copy_engine_gather)
        a.done_counter = self.local.data_ptr() + 4
        ops.tp_fuse(a)
        if pushes:
            self.ag_count += 1
            if self.copy_engine_gather:
                self._copy_rows_to_peers()

    def _copy_rows_to_peers(self) -> None:
        main = torch.cuda.current_stream()
        self.copy_stream.wait_stream(main)
        lo, hi = self.lo, min(self.seq, self.lo + self.rows)
        with torch.cuda.stream(self.copy_stream):
            if hi > lo:
                for r in range(self.world):
                    if r != self.rank:
                        for b in range(self.batch):   # one contiguous block per sample: a plain device-to-device copy
                            self.peer_nbuf[r][b, lo:hi].copy_(self.nbuf[b, lo:hi], non_blocking=True)
            ops.tp_signal(self.ag_flag_ptrs, self.world)

    def join(self) -> None:
        """The main stream waits for the side stream's copies (end of a pass; needed before a capture ends)."""
        torch.cuda.current_stream().wait_stream(self.copy_stream)

    def wait_gathered(self) -> None:
        """Stream-ordered wait until every rank's rows of the latest all-gather sit in the local nbuf."""
        ops.tp_wait(self.flags[self.world:], self.world, self.ag_count, self.epoch_base[1:])
