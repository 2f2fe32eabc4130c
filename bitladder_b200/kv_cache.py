"""A growing low-bit KV cache for one attention layer: what a decoder loop calls.

The reference ships only the two kernels' entry points; its end-to-end cache lives on
a branch that is not part of the project snapshot (``README.md:37``), and its figures
(``imgs/overview.png``, ``imgs/scheme.png``) describe the scheme this class follows:

* tokens are kept unquantized in a tail of at most one pack block (128 tokens at 4 bits,
  256 at 2 bits) per sequence;
* a decode step attends jointly over the packed blocks and the tail
  (``fwd_kvcache_int(..., k_res=, v_res=, res_lens=, cache_seqlens=)``);
* when a sequence's tail is full it is quantized and packed as the next block
  (``kvcache_pack_int(..., dst_token_offset=)``) and the tail starts again.

Everything on the device goes through the two operators of this package; this file is
host logic only.  Lengths are mirrored on the host so that a step needs no
device-to-host synchronisation; in the fused step (``append_and_decode``, ``decoder_step``) the
device keeps them itself, roll-over included, and the mirror is plain arithmetic.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .bit_decode_interface import (alloc_packed_cache, fwd_kvcache_int, kvcache_pack_int, pack_block_tokens)

__all__ = ["PackedKVCache"]


class PackedKVCache:
    """Packed blocks + unquantized tail for ``batch`` sequences of one layer.

    ``max_seqlen`` is the token capacity per sequence (rounded up to whole pack blocks).
    """

    def __init__(self, batch: int, max_seqlen: int, nheads_k: int, head_dim: int = 128, num_bits: int = 4,
                 group_size: int = 128, dtype: torch.dtype = torch.float16, device="cuda"):
        self.batch, self.nheads_k, self.head_dim = batch, nheads_k, head_dim
        self.num_bits, self.group_size, self.dtype = num_bits, group_size, dtype
        self.block = pack_block_tokens(num_bits)
        self.device = torch.device(device)
        self.k_pack, self.k_params, self.v_pack, self.v_params = alloc_packed_cache(
            batch, max_seqlen, nheads_k, head_dim, num_bits, group_size, device=self.device)
        self.capacity = self.v_pack.shape[1]
        self.k_tail = torch.zeros(batch, self.block, nheads_k, head_dim, dtype=dtype, device=self.device)
        self.v_tail = torch.zeros_like(self.k_tail)
        # lengths: host mirror (exact) and device copies the decode kernel reads
        self._packed: List[int] = [0] * batch
        self._tail: List[int] = [0] * batch
        self.cache_seqlens = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.res_lens = torch.zeros(batch, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ lengths
    def seqlens(self) -> List[int]:
        """Tokens held per sequence (packed + tail)."""
        return [p + t for p, t in zip(self._packed, self._tail)]

    def _push_lengths(self) -> None:
        self.cache_seqlens.copy_(torch.tensor(self._packed, dtype=torch.int32), non_blocking=True)
        self.res_lens.copy_(torch.tensor(self._tail, dtype=torch.int32), non_blocking=True)

    # ------------------------------------------------------------------ filling
    def prefill(self, k: torch.Tensor, v: torch.Tensor, seqlens: Optional[Sequence[int]] = None) -> None:
        """Load the prompt's K/V ``(batch, s, nheads_k, head_dim)``: whole blocks are packed, the
        rest goes to the tail.  ``seqlens`` gives per-sequence prompt lengths (default: all ``s``);
        rows beyond a sequence's length are ignored."""
        if k.shape != v.shape or k.dim() != 4 or k.shape[0] != self.batch or k.shape[2:] != (self.nheads_k, self.head_dim):
            raise RuntimeError("prefill expects k and v of shape (batch, s, nheads_k, head_dim)")
        if k.dtype != self.dtype or v.dtype != self.dtype:
            raise RuntimeError(f"prefill expects {self.dtype} tensors")
        s = k.shape[1]
        lens = [s] * self.batch if seqlens is None else [int(x) for x in seqlens]
        if len(lens) != self.batch or any(n < 0 or n > s for n in lens):
            raise RuntimeError("seqlens must hold one length in [0, s] per sequence")
        if any(n > self.capacity for n in lens):
            raise RuntimeError("prompt longer than the cache capacity")
        nb = self.block
        if len(set(lens)) == 1:                       # one launch for the whole batch
            full = lens[0] // nb * nb
            if full:
                kvcache_pack_int(k[:, :full], self.k_pack, self.k_params, v[:, :full], self.v_pack, self.v_params,
                                 None, None, full, "k-channel", self.group_size, self.num_bits)
        else:
            for ib, n in enumerate(lens):
                full = n // nb * nb
                if full:
                    kvcache_pack_int(k[ib:ib + 1, :full], self.k_pack[ib:ib + 1], self.k_params[ib:ib + 1],
                                     v[ib:ib + 1, :full], self.v_pack[ib:ib + 1], self.v_params[ib:ib + 1],
                                     None, None, full, "k-channel", self.group_size, self.num_bits)
        for ib, n in enumerate(lens):
            full = n // nb * nb
            rest = n - full
            if rest:
                self.k_tail[ib, :rest].copy_(k[ib, full:n])
                self.v_tail[ib, :rest].copy_(v[ib, full:n])
            self._packed[ib], self._tail[ib] = full, rest
        self._push_lengths()

    def _roll_full_tails(self) -> None:
        """Pack every tail that is full as its sequence's next block (one ``kvcache_pack_int`` call per
        sequence that rolls over, one for the whole batch when all do at the same length)."""
        nb = self.block
        full = [ib for ib in range(self.batch) if self._tail[ib] == nb]
        if not full:
            return
        if any(self._packed[ib] + nb > self.capacity for ib in full):
            raise RuntimeError("cache capacity exceeded")
        same = len(full) == self.batch and len({self._packed[ib] for ib in full}) == 1
        groups = [list(range(self.batch))] if same else [[ib] for ib in full]
        for grp in groups:
            lo, hi = grp[0], grp[-1] + 1
            kvcache_pack_int(self.k_tail[lo:hi], self.k_pack[lo:hi], self.k_params[lo:hi],
                             self.v_tail[lo:hi], self.v_pack[lo:hi], self.v_params[lo:hi],
                             None, None, nb, "k-channel", self.group_size, self.num_bits,
                             dst_token_offset=self._packed[lo])
        for ib in full:
            self._packed[ib] += nb
            self._tail[ib] = 0
        self._push_lengths()

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """Add one token per sequence, ``(batch, 1, nheads_k, head_dim)``.  A tail that is full is
        packed first."""
        if k_new.shape != (self.batch, 1, self.nheads_k, self.head_dim) or v_new.shape != k_new.shape:
            raise RuntimeError("append expects (batch, 1, nheads_k, head_dim)")
        self._roll_full_tails()
        if len(set(self._tail)) == 1:                 # every sequence writes the same tail slot
            t = self._tail[0]
            self.k_tail[:, t:t + 1].copy_(k_new)
            self.v_tail[:, t:t + 1].copy_(v_new)
        else:
            for ib in range(self.batch):
                t = self._tail[ib]
                self.k_tail[ib, t].copy_(k_new[ib, 0])
                self.v_tail[ib, t].copy_(v_new[ib, 0])
        for ib in range(self.batch):
            self._tail[ib] += 1
        self._push_lengths()

    # ------------------------------------------------------------------ attention
    def decode(self, q: torch.Tensor, softmax_scale: float, **kw) -> torch.Tensor:
        """One decode-attention step of ``q (batch, 1, nheads, head_dim)`` over everything held."""
        seq_hi = max(self._packed) if self._packed else 0
        tail_hi = max(max(self._tail), 1)
        return fwd_kvcache_int(q, self.k_pack, self.k_params, self.v_pack, self.v_params, None, softmax_scale,
                               "k-channel", self.group_size, self.num_bits,
                               k_res=self.k_tail[:, :tail_hi], v_res=self.v_tail[:, :tail_hi],
                               res_lens=self.res_lens, cache_seqlens=self.cache_seqlens,
                               seqlen_k=max(seq_hi, self.block), **kw)

    def _advance_mirror(self) -> None:
        """What the device did to the lengths in a step with ``advance``: pure host arithmetic."""
        for ib in range(self.batch):
            self._tail[ib] += 1
            if self._tail[ib] == self.block and self._packed[ib] + self.block <= self.capacity:
                self._packed[ib] += self.block
                self._tail[ib] = 0

    def append_and_decode(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, softmax_scale: float,
                          **kw) -> torch.Tensor:
        """The decoder's step: attend over everything held plus this step's token ``k_new``/``v_new
        (batch, 1, nheads_k, head_dim)``, leave the token in the tail, and, where a tail has filled up,
        quantize-pack it as the sequence's next block: all on the device (``advance``), no host-side
        packing call, no synchronisation."""
        if k_new.shape != (self.batch, 1, self.nheads_k, self.head_dim) or v_new.shape != k_new.shape:
            raise RuntimeError("append_and_decode expects k_new/v_new of shape (batch, 1, nheads_k, head_dim)")
        self._roll_full_tails()                        # only after plain append() calls left a tail full
        if any(p + t + 1 > self.capacity for p, t in zip(self._packed, self._tail)):
            raise RuntimeError("cache capacity exceeded")
        seq_hi = max(self._packed) if self._packed else 0
        out = fwd_kvcache_int(q, self.k_pack, self.k_params, self.v_pack, self.v_params, None, softmax_scale,
                              "k-channel", self.group_size, self.num_bits,
                              k_res=self.k_tail, v_res=self.v_tail, res_lens=self.res_lens,
                              cache_seqlens=self.cache_seqlens, seqlen_k=max(seq_hi, self.block),
                              k_new=k_new, v_new=v_new, advance=True, **kw)
        self._advance_mirror()
        return out

    def decoder_step(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, softmax_scale: float, **kw):
        """A prepared ``DecodeStep`` that does what ``append_and_decode`` does, for a decoder loop that
        replays a CUDA graph: ``q``, ``k_new`` and ``v_new`` are the buffers the loop refills every step;
        ``step()`` launches the kernels and nothing else (lengths live on the device).  Call
        ``note_steps(n)`` after n steps (or ``sync_lengths()``) before using the other methods again."""
        from .bit_decode_interface import DecodeStep
        self._roll_full_tails()
        return DecodeStep(q, self.k_pack, self.k_params, self.v_pack, self.v_params, None, softmax_scale, "k-channel",
                          self.group_size, self.num_bits, k_res=self.k_tail, v_res=self.v_tail, res_lens=self.res_lens,
                          cache_seqlens=self.cache_seqlens, k_new=k_new, v_new=v_new, advance=True, **kw)

    def note_steps(self, n: int) -> None:
        """Tell the host mirrors that ``n`` steps of a ``decoder_step`` object have been launched."""
        for _ in range(n):
            self._advance_mirror()

    def sync_lengths(self) -> None:
        """Read the lengths back from the device (synchronises)."""
        self._packed = [int(x) for x in self.cache_seqlens.tolist()]
        self._tail = [int(x) for x in self.res_lens.tolist()]
