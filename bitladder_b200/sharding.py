"""Multi-GPU use of the decode path: one process per GPU, `torch.distributed` for plumbing.

The path shards without any data-path collective along the batch and along KV
heads: every (sequence, KV head) pair is independent (it is grid.z of the
reference's split kernel, ``csrc/bit_decode/src/flash_fwd_launch_template.h:110``).
Only when ONE long sequence is split along its tokens is there an exchange step:
each rank attends over its token range and the ranks merge their partial
``(out, lse)`` with the log-sum-exp rule of the reference's split combine
(``csrc/bit_decode/src/flash_fwd_kernel.h:1217-1231, 1280-1298``).  The exchange is
tiny (``b*h*129*4`` bytes per rank) and latency-bound; it is an all-gather (NCCL
on GPUs, gloo in the CPU tests) followed by the local ``bd_combine`` kernel.

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
           "gather_partials", "decode_sequence_parallel", "SequenceParallelStep"]


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


class SequenceParallelStep:
    """``decode_sequence_parallel`` prepared once for a decoder loop: the local partial, the gathered
    partials of all ranks and the result live in buffers allocated here, the local step is a
    ``DecodeStep``, the exchange is ONE ``all_gather_into_tensor`` of ``b*h*(d+1)`` fp32 values per rank
    (each rank's normalised output rows followed by their log-sum-exps) and the merge one ``bd_combine``
    launch over pointers into the gathered buffer.  ``step()`` returns the full result on every rank."""

    def __init__(self, q, k_pack, k_params, v_pack, v_params, softmax_scale, group_size=128, num_bits=4, *,
                 seqlen_k=None, k_res=None, v_res=None, res_lens=None, cache_seqlens=None, group=None,
                 out_dtype=None):
        import torch.distributed as dist

        self._dist, self._group = dist, group
        world = dist.get_world_size(group)
        if world > _lib.BD_MAX_PARTS:
            raise RuntimeError(f"at most {_lib.BD_MAX_PARTS} ranks can share a sequence")
        b, _, h, d = q.shape
        n_out, n = b * h * d, b * h * (d + 1)
        dev = q.device
        self._local = torch.empty(n, dtype=torch.float32, device=dev)
        self._gathered = torch.empty(world * n, dtype=torch.float32, device=dev)
        self._local_step = DecodeStep(q, k_pack, k_params, v_pack, v_params, None, softmax_scale, "k-channel",
                                      group_size, num_bits, seqlen_k=seqlen_k, k_res=k_res, v_res=v_res,
                                      res_lens=res_lens, cache_seqlens=cache_seqlens,
                                      out=self._local[:n_out].view(b, 1, h, d), lse=self._local[n_out:])
        self.out = torch.empty((b, 1, h, d), dtype=out_dtype or q.dtype, device=dev)
        base = self._gathered.data_ptr()
        self._po = (C.c_void_p * world)(*[base + 4 * (r * n) for r in range(world)])
        self._pl = (C.c_void_p * world)(*[base + 4 * (r * n + n_out) for r in range(world)])
        self._args = _lib.CombineArgs(n_parts=world, part_out=C.cast(self._po, C.POINTER(C.c_void_p)),
                                      part_lse=C.cast(self._pl, C.POINTER(C.c_void_p)), rows=b * h, d=d,
                                      out=self.out.data_ptr(), lse=None, out_dtype=_dtype_code(self.out.dtype))
        self._dev = dev

    def step(self):
        self._local_step.step()
        self._dist.all_gather_into_tensor(self._gathered, self._local, group=self._group)
        _lib.check(_lib.load().bd_combine(C.byref(self._args), _stream(self._dev)), "bd_combine")
        return self.out
