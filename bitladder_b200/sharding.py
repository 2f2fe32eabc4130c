"""Multi-GPU use of the decode path: one process per GPU, `torch.distributed` for plumbing.

The path shards without any data-path collective along the batch and along KV
heads: every (sequence, KV head) pair is independent (it is grid.z of the
reference's split kernel, ``csrc/bit_decode/src/flash_fwd_launch_template.h:110``).
Only when ONE long sequence is split along its tokens is there an exchange step:
each rank attends over its token range and the ranks merge their partial
``(out, lse)`` with the log-sum-exp rule of the reference's split combine
(``csrc/bit_decode/src/flash_fwd_kernel.h:1217-1231, 1280-1298``).  The exchange is
tiny (about a kilobyte per (sequence, query head) row and rank) and latency-bound.  On GPUs
it is one kernel per rank behind the decode kernel (``PeerExchange`` / ``bd_decode_exchange``):
it merges the rank's own parts, stores the rows into the peers' memory (value and step counter
side by side, so that no fence or flag is needed), polls for theirs and merges; the portable form
is an all-gather (NCCL, or gloo in the CPU tests) followed by the local ``bd_combine`` kernel.

Nothing here allocates per step beyond the gathered partials; the helpers that
slice caches are meant for set-up time.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

import ctypes as C

from . import _lib
from .bit_decode_interface import (DecodeStep, _dtype_code, _stream, combine_partials, fwd_kvcache_int,
                                   pack_block_tokens)

__all__ = ["shard_range", "shard_batch", "shard_kv_heads", "sequence_shard_bounds",
           "gather_partials", "decode_sequence_parallel", "SequenceParallelStep", "PeerExchange"]


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced [start, stop) of ``n`` items for ``rank`` of ``world``."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(tensors: Sequence[Optional[torch.Tensor]], rank: int, world: int) -> List[Optional[torch.Tensor]]:
    """Slice dim 0 (the batch) of every tensor for this rank; views, no copies."""
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        lo, hi = shard_range(t.shape[0], rank, world)
        out.append(t[lo:hi])
    return out


def shard_kv_heads(q: torch.Tensor, k_pack: torch.Tensor, k_params: torch.Tensor, v_pack: torch.Tensor,
                   v_params: torch.Tensor, rank: int, world: int):
    """This rank's KV heads and the query heads that read them (tensor-parallel style).

    Returns contiguous copies (the packed buffers must be dense in their last three
    dimensions for the kernels), so call it once at set-up, not per step."""
    h_k = k_pack.shape[2]
    h = q.shape[2]
    if h % h_k or h_k % world:
        raise ValueError("KV heads must divide query heads, and the world size must divide KV heads")
    gq = h // h_k
    lo, hi = shard_range(h_k, rank, world)
    return (q[:, :, lo * gq:hi * gq].contiguous(), k_pack[:, :, lo:hi].contiguous(),
            k_params[:, :, lo:hi].contiguous(), v_pack[:, :, lo:hi].contiguous(),
            v_params[:, :, lo:hi].contiguous())


def sequence_shard_bounds(seqlen: int, world: int, num_bits: int) -> List[Tuple[int, int]]:
    """Token ranges for a sequence split over ``world`` ranks, aligned to pack blocks
    (the last range takes the remainder; ranges may be empty for short sequences)."""
    nb = pack_block_tokens(num_bits)
    nblk = (seqlen + nb - 1) // nb
    bounds = []
    for r in range(world):
        lo, hi = shard_range(nblk, r, world)
        bounds.append((min(lo * nb, seqlen), min(hi * nb, seqlen)))
    return bounds


def gather_partials(out_f32: torch.Tensor, lse: torch.Tensor, group=None):
    """All-gather each rank's partial ``(out, lse)``; returns two lists ordered by rank."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    outs = [torch.empty_like(out_f32) for _ in range(world)]
    lses = [torch.empty_like(lse) for _ in range(world)]
    dist.all_gather(outs, out_f32.contiguous(), group=group)
    dist.all_gather(lses, lse.contiguous(), group=group)
    return outs, lses


def decode_sequence_parallel(q, k_pack, k_params, v_pack, v_params, softmax_scale, group_size=128, num_bits=4,
                             *, seqlen_k=None, k_res=None, v_res=None, group=None, out_dtype=None,
                             return_lse=False):
    """One decode step when each rank holds a token range of the SAME sequences.

    Every rank passes its local packed shard (and, on the rank that holds the end of
    the sequence, the unquantized tail); q is replicated.  Each rank computes a
    normalised fp32 partial and its log-sum-exp, the partials are all-gathered and
    merged locally, so every rank returns the full result."""
    out_p, lse_p = fwd_kvcache_int(q, k_pack, k_params, v_pack, v_params, None, softmax_scale, "k-channel",
                                   group_size, num_bits, seqlen_k=seqlen_k, k_res=k_res, v_res=v_res,
                                   out_dtype=torch.float32, return_lse=True)
    outs, lses = gather_partials(out_p, lse_p, group)
    return combine_partials(outs, lses, out_dtype=out_dtype or q.dtype, return_lse=return_lse)


class PeerExchange:
    """The exchange areas of a sequence split, one per rank, mapped into every rank (CUDA IPC).

    Set-up only: ``PeerExchange(rows, group)`` allocates this rank's area through the library
    (``bd_peer_alloc``), passes its 64-byte handle to the other ranks with an ``all_gather_object`` (host
    side, any backend) and maps theirs.  One process per GPU.  ``close()`` unmaps and frees; call it
    with all ranks quiesced."""

    def __init__(self, rows: int, group=None, device=None):
        import torch.distributed as dist

        lib = _lib.load()
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > _lib.BD_MAX_PARTS:
            raise RuntimeError(f"at most {_lib.BD_MAX_PARTS} ranks can share a sequence")
        self.rows = rows
        self._dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.bytes = int(lib.bd_exchange_area_bytes(self.world, rows))
        with torch.cuda.device(self._dev):
            mine = C.c_void_p()
            _lib.check(lib.bd_peer_alloc(self.bytes, C.byref(mine)), "bd_peer_alloc")
            handle = (C.c_ubyte * 64)()
            _lib.check(lib.bd_peer_export(mine, handle), "bd_peer_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.areas = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.areas.append(mine.value)
                    continue
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                ptr = C.c_void_p()
                _lib.check(lib.bd_peer_open(buf, C.byref(ptr)), "bd_peer_open")
                self.areas.append(ptr.value)
        self._mine = mine.value
        self.c_areas = (C.c_void_p * self.world)(*self.areas)
        self._group = group

    def state(self):
        """Wait for the current stream; returns (status, epoch) of this rank's area and clears the status."""
        epoch = C.c_uint32()
        with torch.cuda.device(self._dev):
            rc = int(_lib.load().bd_exchange_state(self._mine, _stream(self._dev), C.byref(epoch)))
        return rc, int(epoch.value)

    def close(self):
        lib = _lib.load()
        with torch.cuda.device(self._dev):
            torch.cuda.synchronize()
            for r, ptr in enumerate(self.areas):
                if ptr is None:
                    continue
                if r == self.rank:
                    lib.bd_peer_free(ptr)
                else:
                    lib.bd_peer_close(ptr)
        self.areas = [None] * self.world


class SequenceParallelStep:
    """``decode_sequence_parallel`` prepared once for a decoder loop.

    * ``exchange="peer"`` (default on GPUs): the step is ``bd_decode_exchange``: the decode kernel over this
      rank's shard leaves its CTAs' parts in the workspace, and ONE more kernel merges them row by row,
      stores each row into every peer's exchange area over NVLink (values and the step's epoch side by
      side, no fence or flag), polls (bounded) for the peers' rows in its own area and merges them.
      Two launches per step, no NCCL call, nothing allocated, capturable in a CUDA graph
      (``capturable``).  A peer that does not publish makes the kernel give up after ``spin_limit`` polls
      and leave ``BD_ERR_TIMEOUT`` in the area's status word (``check()`` raises then).
    * ``exchange="nccl"``: the local step is a ``DecodeStep`` that writes this rank's fp32 partial and its
      log-sum-exps, then one ``all_gather_into_tensor`` of ``b*h*(d+1)`` fp32 values per rank and one
      ``bd_combine`` launch over pointers into the gathered buffer.

    ``step()`` returns the full result on every rank."""

    def __init__(self, q, k_pack, k_params, v_pack, v_params, softmax_scale, group_size=128, num_bits=4, *,
                 seqlen_k=None, k_res=None, v_res=None, res_lens=None, cache_seqlens=None, group=None,
                 out_dtype=None, exchange="peer", spin_limit=0):
        import torch.distributed as dist

        self._dist, self._group = dist, group
        world = dist.get_world_size(group)
        if world > _lib.BD_MAX_PARTS:
            raise RuntimeError(f"at most {_lib.BD_MAX_PARTS} ranks can share a sequence")
        b, _, h, d = q.shape
        rows = b * h
        n_out = rows * d
        lse_off = (n_out + 3) // 4 * 4                 # both parts of a rank's record start on 16 bytes
        n = lse_off + (rows + 3) // 4 * 4
        dev = q.device
        self._dev = dev
        self.out = torch.empty((b, 1, h, d), dtype=out_dtype or q.dtype, device=dev)
        self.kind = exchange
        if exchange == "peer":
            # the decode step writes nothing final itself: out receives the merged result of all ranks
            self._local_step = DecodeStep(q, k_pack, k_params, v_pack, v_params, None, softmax_scale, "k-channel",
                                          group_size, num_bits, seqlen_k=seqlen_k, k_res=k_res, v_res=v_res,
                                          res_lens=res_lens, cache_seqlens=cache_seqlens, out=self.out)
            self.peers = PeerExchange(rows, group, dev)
            self._xargs = _lib.ExchangeArgs(rank=self.peers.rank, world=world,
                                            areas=C.cast(self.peers.c_areas, C.POINTER(C.c_void_p)),
                                            part_out=None, part_lse=None, rows=rows, d=d, out=None, lse=None,
                                            out_dtype=_dtype_code(self.out.dtype), spin_limit=int(spin_limit))
            self.capturable = True
            self.exchange = {"kind": "rows stored into the peers' mapped exchange areas (value + epoch in every 8 bytes), "
                                     "local parts merge, exchange and final merge in one kernel",
                             "launches": 1, "merges_local_parts": True,
                             "bytes_per_rank_per_peer": rows * (d // 2 + 1) * 16}
        elif exchange == "nccl":
            self._local = torch.empty(n, dtype=torch.float32, device=dev)
            self._local_step = DecodeStep(q, k_pack, k_params, v_pack, v_params, None, softmax_scale, "k-channel",
                                          group_size, num_bits, seqlen_k=seqlen_k, k_res=k_res, v_res=v_res,
                                          res_lens=res_lens, cache_seqlens=cache_seqlens,
                                          out=self._local[:n_out].view(b, 1, h, d), lse=self._local[lse_off:lse_off + rows])
            self._gathered = torch.empty(world * n, dtype=torch.float32, device=dev)
            base = self._gathered.data_ptr()
            self._po = (C.c_void_p * world)(*[base + 4 * (r * n) for r in range(world)])
            self._pl = (C.c_void_p * world)(*[base + 4 * (r * n + lse_off) for r in range(world)])
            self._args = _lib.CombineArgs(n_parts=world, part_out=C.cast(self._po, C.POINTER(C.c_void_p)),
                                          part_lse=C.cast(self._pl, C.POINTER(C.c_void_p)), rows=rows, d=d,
                                          out=self.out.data_ptr(), lse=None, out_dtype=_dtype_code(self.out.dtype))
            self.capturable = False
            self.exchange = {"kind": "NCCL all_gather_into_tensor + bd_combine", "launches": 2,
                             "bytes_per_rank_per_peer": 4 * n}
        else:
            raise ValueError("exchange must be 'peer' or 'nccl'")

    def step(self):
        with torch.cuda.device(self._dev):
            if self.kind == "peer":
                _lib.check(_lib.load().bd_decode_exchange(self._local_step._ref, C.byref(self._xargs), _stream(self._dev)),
                           "bd_decode_exchange")
            else:
                self._local_step.step()
                self._dist.all_gather_into_tensor(self._gathered, self._local, group=self._group)
                _lib.check(_lib.load().bd_combine(C.byref(self._args), _stream(self._dev)), "bd_combine")
        return self.out

    def check(self):
        """Wait for the stream and raise if a step's exchange gave up waiting for a peer."""
        if self.kind == "peer":
            rc, _ = self.peers.state()
            if rc != 0:
                raise RuntimeError(f"sequence-parallel step failed on the device: {_lib.strerror(rc)} (code {rc})")

    def close(self):
        if self.kind == "peer":
            self.peers.close()
