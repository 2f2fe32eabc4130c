"""Python entry points of the low-bit KV-cache decode-attention path.

Drop-in for the two functions of the reference's ``bit_decode`` package
(reference: ``bit_decode/bit_decode_interface.py:10-41`` ``kvcache_pack_int`` and
``:43-86`` ``fwd_kvcache_int``): same names, same positional arguments, same
caller-allocated buffers with the same shapes and dtypes.  Tensors cross a C-ABI
(``include/bitdecode.h``) as raw device pointers; the kernels are hand-written
CUDA for sm_100a.  There is no CPU or PyTorch fallback: without the built
library, or on a non-CUDA tensor, the calls raise ``RuntimeError``.

Differences from the reference, all of them additions or stricter checks:

* keyword-only extensions on the decode call: an unquantized fp16/bf16 tail
  (``k_res``/``v_res``/``res_lens``), per-sequence lengths (``cache_seqlens``),
  a returned log-sum-exp, a caller-provided output / workspace, fp32 output;
* bf16 inputs and group size 64 are implemented (the reference accepts the
  arguments but has no kernels for them); group size 32 as in the reference;
* unsupported ``(quant_mode, group_size, num_bits, dtype)`` combinations raise
  instead of silently doing nothing (reference: ``csrc/bit_decode/decode_api.cpp:207-226``);
* paged caches (``opt_block_table``): the four packed buffers then hold pages of 256-token
  multiples instead of sequences, as in the reference (``decode_api.cpp:328-352``); the pack
  call packs every page of the pool it is given.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

__all__ = ["kvcache_pack_int", "fwd_kvcache_int", "combine_partials", "decode_workspace_bytes",
           "plan_splits", "pack_block_tokens", "alloc_packed_cache", "DecodeStep"]

_WORKSPACES = {}


def pack_block_tokens(num_bits: int) -> int:
    """Tokens per pack block: K codes are grouped 32 rows x (16 // num_bits) fields."""
    return 32 * (16 // num_bits)


def _dtype_code(t: torch.dtype) -> int:
    if t == torch.float16:
        return _lib.BD_FP16
    if t == torch.bfloat16:
        return _lib.BD_BF16
    if t == torch.float32:
        return _lib.BD_FP32
    raise RuntimeError(f"unsupported dtype {t}: only fp16 and bf16 inputs are supported")


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_cuda(*tensors) -> None:
    dev = None
    for t in tensors:
        if t is None:
            continue
        _require(t.is_cuda, "all tensors must be on a CUDA device (there is no CPU path)")
        dev = dev if dev is not None else t.device
        _require(t.device == dev, "all tensors must be on the same device")


def _check_config(quant_mode: str, group_size: int, num_bits: int) -> None:
    _require(quant_mode == "k-channel", f"quant_mode {quant_mode!r} is not supported (only 'k-channel')")
    _require(num_bits in (2, 4), f"num_bits must be 2 or 4, got {num_bits}")
    _require(group_size in (32, 64, 128), f"group_size must be 32, 64 or 128, got {group_size}")


def _rows_contiguous(t: torch.Tensor) -> bool:
    """True when dims 1.. are laid out densely (dim 0 may have any stride)."""
    expected = 1
    for size, stride in zip(reversed(t.shape[1:]), reversed(t.stride()[1:])):
        if size != 1 and stride != expected:
            return False
        expected *= size
    return True


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def alloc_packed_cache(batch: int, seqlen: int, nheads_k: int, d: int = 128, num_bits: int = 4,
                       group_size: int = 128, device="cuda"):
    """Allocate the four packed buffers with the shapes the reference's callers use
    (reference: ``evaluation/test.py:76-83``).  ``seqlen`` is rounded up to whole pack blocks."""
    nb = pack_block_tokens(num_bits)
    s = (seqlen + nb - 1) // nb * nb
    pn = 16 // num_bits
    k_pack = torch.zeros((batch, s // pn, nheads_k, d), dtype=torch.uint16, device=device)
    k_params = torch.zeros((batch, s // group_size, nheads_k, d), dtype=torch.float32, device=device)
    v_pack = torch.zeros((batch, s, nheads_k, d // pn), dtype=torch.uint16, device=device)
    v_params = torch.zeros((batch, d // group_size, nheads_k, s), dtype=torch.float32, device=device)
    return k_pack, k_params, v_pack, v_params


def _check_packed(k_pack, k_params, v_pack, v_params, num_bits, group_size):
    pn = 16 // num_bits
    nb = pack_block_tokens(num_bits)
    for name, t in (("k_pack", k_pack), ("v_pack", v_pack)):
        _require(t.dtype in (torch.uint16, torch.int16), f"{name} must be uint16")
    for name, t in (("k_params", k_params), ("v_params", v_params)):
        _require(t.dtype == torch.float32, f"{name} must be float32 storage (one fp16 scale + one fp16 zero per slot)")
    for name, t in (("k_pack", k_pack), ("k_params", k_params), ("v_pack", v_pack), ("v_params", v_params)):
        _require(t.dim() == 4, f"{name} must have 4 dimensions")
        _require(_rows_contiguous(t), f"{name} must be contiguous in its last three dimensions")
    b, s_cap, h_k, dp = v_pack.shape
    d = dp * pn
    _require(d == 128, f"head dimension must be 128, got {d}")
    _require(s_cap % nb == 0, f"packed sequence capacity {s_cap} must be a multiple of {nb}")
    _require(tuple(k_pack.shape) == (b, s_cap // pn, h_k, d), "k_pack shape must be (b, s/pack_num, h_k, d)")
    _require(tuple(k_params.shape) == (b, s_cap // group_size, h_k, d), "k_params shape must be (b, s/group, h_k, d)")
    _require(tuple(v_params.shape) == (b, d // group_size, h_k, s_cap), "v_params shape must be (b, d/group, h_k, s)")
    return b, s_cap, h_k, d


def kvcache_pack_int(k_cache: torch.Tensor, k_pack: torch.Tensor, k_params: torch.Tensor,
                     v_cache: torch.Tensor, v_pack: torch.Tensor, v_params: torch.Tensor,
                     opt_block_table: Optional[torch.Tensor] = None,
                     cu_seqlens_k: torch.Tensor = None,
                     seqlen_k: int = 0,
                     quant_mode: str = "k-channel",
                     group_size: int = 128,
                     num_bits: int = 4,
                     *, dst_token_offset: int = 0, reference_fast_math: bool = False) -> None:
    """Quantize ``k_cache``/``v_cache`` (b, s, h_k, d) and pack them in place into
    ``k_pack``/``k_params``/``v_pack``/``v_params``.

    Same signature as the reference (``bit_decode_interface.py:10-41``); like
    there, ``seqlen_k`` is taken from ``k_cache.shape[1]`` and ``cu_seqlens_k`` is
    accepted but not read.  ``dst_token_offset`` (extension) writes the packed
    tokens at that offset of the pack buffers, for caches that grow block by block.
    ``reference_fast_math`` (extension) divides the way the reference does as it is shipped
    (built with ``--use_fast_math``: the GPU's approximate reciprocal), which gives the very bytes
    that build writes on the same GPU; the default is IEEE division, the bytes of the reference
    built without that flag and of a CPU evaluation of its formulas.  The two differ by one code
    step at exact rounding ties, a few codes in 10^5.  Asynchronous on the current stream.
    """
    _check_config(quant_mode, group_size, num_bits)
    # A paged pool is packed page by page: quantization groups never cross a pack block, so the
    # pages are just `num_pages` independent sequences of `page_size` tokens and the table is not needed.
    if opt_block_table is not None:
        _require(k_cache.dim() == 4 and k_cache.shape[1] % 256 == 0, "Paged KV cache block size must be divisible by 256")
    _check_cuda(k_cache, v_cache, k_pack, k_params, v_pack, v_params)
    _require(k_cache.dtype in (torch.float16, torch.bfloat16), "k_cache must be fp16 or bf16")
    _require(v_cache.dtype == k_cache.dtype, "k_cache and v_cache must have the same dtype")
    _require(k_cache.dim() == 4 and k_cache.shape == v_cache.shape, "k_cache and v_cache must both be (b, s, h_k, d)")
    _require(k_cache.stride(-1) == 1 and v_cache.stride(-1) == 1, "Input tensor must have contiguous last dimension")
    b, s, h_k, d = k_cache.shape
    pb, s_cap, ph, pd = _check_packed(k_pack, k_params, v_pack, v_params, num_bits, group_size)
    _require((pb, ph, pd) == (b, h_k, d), "packed buffers do not match k_cache's batch / heads / head_dim")
    nb = pack_block_tokens(num_bits)
    _require(s % nb == 0, f"sequence length {s} must be a multiple of {nb} for {num_bits}-bit packing")
    _require(dst_token_offset % nb == 0 and dst_token_offset >= 0, f"dst_token_offset must be a multiple of {nb}")
    _require(dst_token_offset + s <= s_cap, "packed buffers are too small for this many tokens")
    if s == 0:
        return
    a = _lib.PackArgs(
        k=k_cache.data_ptr(), v=v_cache.data_ptr(),
        k_stride_b=k_cache.stride(0), k_stride_s=k_cache.stride(1), k_stride_h=k_cache.stride(2),
        v_stride_b=v_cache.stride(0), v_stride_s=v_cache.stride(1), v_stride_h=v_cache.stride(2),
        k_pack=k_pack.data_ptr(), k_params=k_params.data_ptr(),
        v_pack=v_pack.data_ptr(), v_params=v_params.data_ptr(),
        k_pack_stride_b=k_pack.stride(0), k_params_stride_b=k_params.stride(0),
        v_pack_stride_b=v_pack.stride(0),
        v_params_stride_b=v_params.stride(0), v_params_stride_g=v_params.stride(1),
        v_params_stride_h=v_params.stride(2),
        b=b, s=s, h_k=h_k, d=d, dst_token_offset=dst_token_offset,
        bits=num_bits, group=group_size, dtype=_dtype_code(k_cache.dtype),
        flags=_lib.BD_PACK_APPROX_DIV if reference_fast_math else 0)
    with torch.cuda.device(k_cache.device):
        _lib.check(_lib.load().bd_pack(C.byref(a), _stream(k_cache.device)), "bd_pack")


def _decode_args(q, k_pack, k_params, v_pack, v_params, softmax_scale, group_size, num_bits,
                 k_res, v_res, res_lens, cache_seqlens, seqlen_k, out, lse, num_splits, block_table=None,
                 k_new=None, v_new=None, spin_limit=0, test_starve=0, advance=False, rotary=None):
    b, s_cap, h_k, d = _check_packed(k_pack, k_params, v_pack, v_params, num_bits, group_size)
    _require(q.dim() == 4 and q.shape[1] == 1, "q must be (b, 1, h, d): one query token per sequence")
    num_pages = 0
    if block_table is not None:
        # paged cache (reference: decode_api.cpp:328-352): the buffers hold pages, not sequences
        _require(block_table.dtype == torch.int32, "block_table must have dtype torch.int32")
        _require(block_table.dim() == 2 and block_table.stride(-1) == 1,
                 "block_table must be (b, max_blocks) with a contiguous last dimension")
        _require(s_cap % 256 == 0, "Paged KV cache block size must be divisible by 256")
        num_pages, b = b, block_table.shape[0]
    _require(q.shape[0] == b and q.shape[3] == d, "q does not match the packed cache's batch / head_dim")
    h = q.shape[2]
    _require(h % h_k == 0, "Number of heads in key/value must divide number of heads in query")
    _require(h // h_k <= 16, "at most 16 query heads per KV head are supported")
    _require(q.stride(-1) == 1, "Input tensor must have contiguous last dimension")
    s_max = s_cap if block_table is None else s_cap * block_table.shape[1]
    s = s_max if seqlen_k is None else int(seqlen_k)
    _require(0 <= s <= s_max, "seqlen_k exceeds the packed buffers")
    a = _lib.DecodeArgs()
    if block_table is not None:
        a.block_table, a.block_table_stride, a.num_pages = block_table.data_ptr(), block_table.stride(0), num_pages
    a.q, a.out, a.lse = q.data_ptr(), out.data_ptr(), (lse.data_ptr() if lse is not None else None)
    a.q_stride_b, a.q_stride_h = q.stride(0), q.stride(2)
    a.out_stride_b, a.out_stride_h = out.stride(0), out.stride(2)
    a.k_pack, a.k_params, a.v_pack, a.v_params = (k_pack.data_ptr(), k_params.data_ptr(),
                                                  v_pack.data_ptr(), v_params.data_ptr())
    a.k_pack_stride_b, a.k_params_stride_b, a.v_pack_stride_b = k_pack.stride(0), k_params.stride(0), v_pack.stride(0)
    a.v_params_stride_b, a.v_params_stride_g, a.v_params_stride_h = (v_params.stride(0), v_params.stride(1),
                                                                     v_params.stride(2))
    if cache_seqlens is not None:
        _require(cache_seqlens.dtype == torch.int32 and cache_seqlens.numel() == b and cache_seqlens.is_contiguous(),
                 "cache_seqlens must be a contiguous int32 tensor of shape (b,)")
        a.cache_seqlens = cache_seqlens.data_ptr()
    if k_res is not None or v_res is not None:
        _require(k_res is not None and v_res is not None, "k_res and v_res must be given together")
        _require(k_res.dtype == q.dtype and v_res.dtype == q.dtype, "the tail must have q's dtype")
        _require(k_res.dim() == 4 and k_res.shape == v_res.shape and k_res.stride() == v_res.stride(),
                 "k_res and v_res must both be (b, r, h_k, d) with equal strides")
        _require(k_res.shape[0] == b and k_res.shape[2] == h_k and k_res.shape[3] == d,
                 "the tail does not match the packed cache's batch / heads / head_dim")
        _require(k_res.shape[1] <= 256, "the unquantized tail holds at most 256 tokens")
        _require(k_res.stride(-1) == 1, "Input tensor must have contiguous last dimension")
        a.k_res, a.v_res = k_res.data_ptr(), v_res.data_ptr()
        a.res_stride_b, a.res_stride_s, a.res_stride_h = k_res.stride(0), k_res.stride(1), k_res.stride(2)
        a.res_len = k_res.shape[1]
        if res_lens is not None:
            _require(res_lens.dtype == torch.int32 and res_lens.numel() == b and res_lens.is_contiguous(),
                     "res_lens must be a contiguous int32 tensor of shape (b,)")
            a.res_lens = res_lens.data_ptr()
    if k_new is not None or v_new is not None:
        _require(k_new is not None and v_new is not None, "k_new and v_new must be given together")
        _require(k_res is not None and res_lens is not None,
                 "k_new/v_new are appended to the tail: k_res, v_res and res_lens are needed")
        _require(k_new.dtype == q.dtype and v_new.dtype == q.dtype, "k_new/v_new must have q's dtype")
        _require(tuple(k_new.shape) == (b, 1, h_k, d) and k_new.shape == v_new.shape and k_new.stride() == v_new.stride(),
                 "k_new and v_new must both be (b, 1, h_k, d) with equal strides")
        _require(k_new.stride(-1) == 1, "Input tensor must have contiguous last dimension")
        a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
        a.new_stride_b, a.new_stride_h = k_new.stride(0), k_new.stride(2)
    a.b, a.h, a.h_k, a.d = b, h, h_k, d
    a.s, a.s_cap = s, s_cap
    a.bits, a.group = num_bits, group_size
    a.dtype, a.out_dtype = _dtype_code(q.dtype), _dtype_code(out.dtype)
    a.softmax_scale = float(softmax_scale)
    a.num_splits = int(num_splits)
    a.spin_limit, a.test_starve = int(spin_limit), int(test_starve)
    if advance:
        _require(k_new is not None and cache_seqlens is not None and res_lens is not None and block_table is None,
                 "advance needs k_new/v_new, cache_seqlens and res_lens, and a cache without a block table")
        _require(k_res.shape[1] >= pack_block_tokens(num_bits),
                 f"advance needs a tail buffer of at least {pack_block_tokens(num_bits)} rows (one pack block)")
        a.advance = 1
    if rotary is not None:
        cos, sin, interleaved = rotary
        _require(k_new is not None, "rotary embedding applies to the appended token: k_new/v_new are needed")
        _require(cos.is_cuda and sin.is_cuda and cos.device == q.device and sin.device == q.device,
                 "rotary_cos / rotary_sin must be CUDA tensors on q's device")
        _require(cos.dtype == q.dtype and sin.dtype == q.dtype, "rotary_cos / rotary_sin must have q's dtype")
        _require(cos.dim() == 2 and cos.shape == sin.shape and cos.is_contiguous() and sin.is_contiguous(),
                 "rotary_cos / rotary_sin must be contiguous (positions, rotary_dim / 2)")
        rotary_dim = 2 * cos.shape[1]
        _require(0 < rotary_dim <= d and rotary_dim % 16 == 0, "rotary_dim must be a multiple of 16, at most head_dim")
        a.rotary_cos, a.rotary_sin = cos.data_ptr(), sin.data_ptr()
        a.rotary_dim, a.rotary_interleaved, a.rotary_positions = rotary_dim, 1 if interleaved else 0, cos.shape[0]
    return a


def _workspace_for(a: "_lib.DecodeArgs", device, workspace):
    need = int(_lib.load().bd_decode_workspace_bytes(C.byref(a)))
    _require(need > 0, "bd_decode_workspace_bytes rejected the arguments")
    if workspace is None:
        # Cached per (device, stream).  The library wants a zeroed workspace and leaves
        # its counters at zero after every call, but their place depends on the batch
        # size and head count: clear the buffer again whenever that layout changes.
        key = (device.index, _stream(device))
        layout = (a.b, a.h_k, a.cache_seqlens is not None)
        entry = _WORKSPACES.get(key)
        if entry is None or entry[0].numel() < need:
            entry = [torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device), layout]
            _WORKSPACES[key] = entry
        elif entry[1] != layout:
            entry[0].zero_()
            entry[1] = layout
        workspace = entry[0]
    else:
        _require(workspace.is_cuda and workspace.dtype == torch.uint8 and workspace.is_contiguous(),
                 "workspace must be a contiguous uint8 CUDA tensor")
        _require(workspace.numel() >= need, f"workspace too small: need {need} bytes")
    a.workspace = workspace.data_ptr()
    a.workspace_bytes = workspace.numel()
    return workspace


def fwd_kvcache_int(q: torch.Tensor,
                    k_pack: torch.Tensor, k_params: torch.Tensor,
                    v_pack: torch.Tensor, v_params: torch.Tensor,
                    opt_block_table: Optional[torch.Tensor] = None,
                    softmax_scale: float = 1.0,
                    quant_mode: str = "k-channel",
                    group_size: int = 128,
                    num_bits: int = 4,
                    *, k_res: Optional[torch.Tensor] = None, v_res: Optional[torch.Tensor] = None,
                    res_lens: Optional[torch.Tensor] = None, cache_seqlens: Optional[torch.Tensor] = None,
                    seqlen_k: Optional[int] = None, return_lse: bool = False,
                    out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                    workspace: Optional[torch.Tensor] = None, num_splits: int = 0,
                    k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
                    check: bool = False, spin_limit: int = 0, _test_starve: int = 0, advance: bool = False,
                    rotary_cos: Optional[torch.Tensor] = None, rotary_sin: Optional[torch.Tensor] = None,
                    rotary_interleaved: bool = True):
    """One decode-attention step over the packed cache; returns ``out`` (b, 1, h, d).

    Same positional signature as the reference (``bit_decode_interface.py:43-86``),
    which hard-wires non-causal, no window, no softcap and automatic splits; so does
    this one.  Keyword-only extensions: ``k_res``/``v_res`` (b, r<=256, h_k, d)
    unquantized tail attended jointly with the packed tokens (``res_lens`` int32 (b,)
    gives per-sequence tail lengths); ``cache_seqlens`` int32 (b,) per-sequence count
    of packed tokens; ``seqlen_k`` upper bound on packed tokens (default: the
    buffers' capacity, like the reference's ``v_pack.size(1)``); ``return_lse``
    also returns the (b, h) fp32 log-sum-exp of the scaled scores; ``out`` /
    ``out_dtype`` (fp16, bf16 or fp32) / ``workspace`` / ``num_splits`` for callers
    that manage memory and scheduling themselves (a caller-provided ``workspace`` must
    be zero-filled once, and again whenever the batch size or KV head count it is used
    with changes); ``k_new``/``v_new`` (b, 1, h_k, d): the K/V rows of the token decoded in this
    step — the step attends over them as the next tail row and stores them at row ``res_lens[b]`` of
    ``k_res``/``v_res`` (fused append; the caller then adds one to ``res_lens``, which must be below
    the tail buffers' length); with ``advance=True`` the library does that bookkeeping on the device
    instead: after the step ``res_lens`` is one larger, and a tail that has reached one pack block is
    quantize-packed as the sequence's next block, ``cache_seqlens`` grows by that block and ``res_lens``
    starts again at 0 (the roll-over of the reference's residual scheme), so a decoder step needs no host
    logic and can be captured in a CUDA graph; ``rotary_cos``/``rotary_sin`` (positions, rotary_dim / 2, q's dtype),
    with ``k_new``: q and k_new are rotated at the token's position ``cache_seqlens[b] + res_lens[b]`` first (pairs
    (2i, 2i+1) if ``rotary_interleaved`` else (i, i + rotary_dim/2); the reference's dormant append path,
    ``decode_api.cpp:316, 418``, ``src/include/flash.h:149-151``), so the rotated key is what the step attends over and files in the tail.
    Asynchronous on the current stream, unless ``check=True``: then the
    call waits for the step and raises ``RuntimeError`` if the kernel reported an error (a device-side
    wait on a copy that ran out after ``spin_limit`` polls, 0 = the library's default of seconds; a
    ``opt_block_table`` entry outside the page pool).  Without ``check`` such a step returns
    unusable values silently; a serving loop checks every n-th step.
    """
    _check_config(quant_mode, group_size, num_bits)
    _check_cuda(q, k_pack, k_params, v_pack, v_params, k_res, v_res, res_lens, cache_seqlens, out, workspace,
                opt_block_table, k_new, v_new)
    _require(q.dtype in (torch.float16, torch.bfloat16), "q must be fp16 or bf16")
    if out is None:
        out = torch.empty(q.shape, dtype=out_dtype or q.dtype, device=q.device)
    else:
        _require(out.shape == q.shape and out.stride(-1) == 1, "out must have q's shape and a contiguous last dimension")
    lse = torch.empty((q.shape[0], q.shape[2]), dtype=torch.float32, device=q.device) if return_lse else None
    _require((rotary_cos is None) == (rotary_sin is None), "rotary_cos and rotary_sin must be given together")
    rotary = None if rotary_cos is None else (rotary_cos, rotary_sin, rotary_interleaved)
    a = _decode_args(q, k_pack, k_params, v_pack, v_params, softmax_scale, group_size, num_bits,
                     k_res, v_res, res_lens, cache_seqlens, seqlen_k, out, lse, num_splits, opt_block_table,
                     k_new, v_new, spin_limit, _test_starve, advance, rotary)
    with torch.cuda.device(q.device):
        ws = _workspace_for(a, q.device, workspace)
        _lib.check(_lib.load().bd_decode(C.byref(a), _stream(q.device)), "bd_decode")
        if check:
            _check_status(ws, q.device)
    del ws
    return (out, lse) if return_lse else out


def _check_status(workspace: torch.Tensor, device) -> None:
    """Wait for the stream and raise if a decode kernel left an error in the workspace's status word."""
    rc = int(_lib.load().bd_read_status(workspace.data_ptr(), _stream(device)))
    if rc != 0:
        workspace.zero_()                 # counters may be anywhere after an aborted step
        raise RuntimeError(f"decode step failed on the device: {_lib.strerror(rc)} (code {rc})")


class DecodeStep:
    """One decode-attention step, checked and laid out once, launched many times.

    ``fwd_kvcache_int`` validates its tensors and fills the C argument block on every call,
    some tens of microseconds of Python around a kernel of about sixty.  A decoder loop calls
    with the same buffers every step (the query buffer, the cache, the tail, the length
    tensors all stay where they are and only their contents change), so this class does that
    work once: it takes the same arguments as ``fwd_kvcache_int``, keeps the tensors alive,
    owns its output (and LSE) buffer and a private zeroed workspace, and ``step()`` is one
    call into the library on the current stream.  Contents may change between steps
    (``q.copy_(...)``, ``res_lens += 1``, new rows in the tail); addresses, shapes and strides
    may not — build a new object when they do.
    """

    def __init__(self, q, k_pack, k_params, v_pack, v_params, opt_block_table=None, softmax_scale=1.0,
                 quant_mode="k-channel", group_size=128, num_bits=4, *, k_res=None, v_res=None, res_lens=None,
                 cache_seqlens=None, seqlen_k=None, return_lse=False, out=None, out_dtype=None, num_splits=0,
                 k_new=None, v_new=None, lse=None, spin_limit=0, _test_starve=0, advance=False,
                 rotary_cos=None, rotary_sin=None, rotary_interleaved=True):
        _check_config(quant_mode, group_size, num_bits)
        _check_cuda(q, k_pack, k_params, v_pack, v_params, k_res, v_res, res_lens, cache_seqlens, out,
                    opt_block_table, k_new, v_new)
        _require(q.dtype in (torch.float16, torch.bfloat16), "q must be fp16 or bf16")
        if out is None:
            out = torch.empty(q.shape, dtype=out_dtype or q.dtype, device=q.device)
        else:
            _require(out.shape == q.shape and out.stride(-1) == 1,
                     "out must have q's shape and a contiguous last dimension")
        self.out = out
        if lse is not None:
            _require(lse.is_cuda and lse.dtype == torch.float32 and lse.is_contiguous() and
                     lse.numel() == q.shape[0] * q.shape[2], "lse must be a contiguous fp32 CUDA tensor of b*h elements")
            self.lse = lse
        else:
            self.lse = (torch.empty((q.shape[0], q.shape[2]), dtype=torch.float32, device=q.device)
                        if return_lse else None)
        _require((rotary_cos is None) == (rotary_sin is None), "rotary_cos and rotary_sin must be given together")
        rotary = None if rotary_cos is None else (rotary_cos, rotary_sin, rotary_interleaved)
        self._args = _decode_args(q, k_pack, k_params, v_pack, v_params, softmax_scale, group_size, num_bits,
                                  k_res, v_res, res_lens, cache_seqlens, seqlen_k, out, self.lse, num_splits,
                                  opt_block_table, k_new, v_new, spin_limit, _test_starve, advance, rotary)
        self._device = q.device
        with torch.cuda.device(q.device):
            need = int(_lib.load().bd_decode_workspace_bytes(C.byref(self._args)))
            _require(need > 0, "bd_decode_workspace_bytes rejected the arguments")
            self._workspace = torch.zeros(need, dtype=torch.uint8, device=q.device)
        self._args.workspace, self._args.workspace_bytes = self._workspace.data_ptr(), need
        self._keep = (q, k_pack, k_params, v_pack, v_params, opt_block_table, k_res, v_res, res_lens, cache_seqlens,
                      k_new, v_new, rotary_cos, rotary_sin)
        self._fn = _lib.load().bd_decode
        self._ref = C.byref(self._args)

    def step(self, check: bool = False):
        """Launch the step on the current stream of the tensors' device; returns ``out`` (or
        ``(out, lse)``), the same buffers every time.  ``check=True`` waits for the step and raises
        ``RuntimeError`` if the kernel reported an error (see ``fwd_kvcache_int``); it synchronises,
        so a loop uses it every n-th step, and never inside a stream capture."""
        if torch.cuda.current_device() != self._device.index:
            with torch.cuda.device(self._device):
                rc = self._fn(self._ref, _stream(self._device))
        else:
            rc = self._fn(self._ref, _stream(self._device))
        if rc != 0:
            _lib.check(rc, "bd_decode")
        if check:
            with torch.cuda.device(self._device):
                _check_status(self._workspace, self._device)
        return (self.out, self.lse) if self.lse is not None else self.out

    def plan(self) -> dict:
        """How the library runs this step on the tensors' device: ranges per KV head (``rows``), CTAs
        resident per SM, streaming warps per CTA and kernels launched per step."""
        out = (C.c_int32 * 4)()
        with torch.cuda.device(self._device):
            _lib.check(_lib.load().bd_decode_plan(self._ref, out), "bd_decode_plan")
        return {"rows": int(out[0]), "ctas_per_sm": int(out[1]), "warps_per_cta": int(out[2]), "launches": int(out[3])}

    def status(self) -> int:
        """Wait for the stream; return (and clear) the error code the steps so far left: 0 for none."""
        with torch.cuda.device(self._device):
            return int(_lib.load().bd_read_status(self._workspace.data_ptr(), _stream(self._device)))


def decode_workspace_bytes(q, k_pack, k_params, v_pack, v_params, group_size=128, num_bits=4,
                           seqlen_k=None, num_splits=0, k_res=None, v_res=None, res_lens=None,
                           cache_seqlens=None, block_table=None) -> int:
    """Bytes of workspace a decode call with these tensors needs (the tail and
    per-sequence lengths add to it, so pass them if the call will)."""
    a = _decode_args(q, k_pack, k_params, v_pack, v_params, 1.0, group_size, num_bits,
                     k_res, v_res, res_lens, cache_seqlens, seqlen_k, q, None, num_splits, block_table)
    with torch.cuda.device(q.device):
        return int(_lib.load().bd_decode_workspace_bytes(C.byref(a)))


def plan_splits(batch: int, nheads_k: int, max_seqlen: int, num_bits: int = 4, sm_count: int = 148,
                ctas_per_sm: int = 0) -> int:
    """Sequence splits the decode call picks on a device with ``sm_count`` SMs (pure host logic)."""
    return int(_lib.load().bd_plan_splits(batch, nheads_k, max_seqlen, num_bits, sm_count, ctas_per_sm))


def combine_partials(part_outs, part_lses, out_dtype: torch.dtype = torch.float16, return_lse: bool = False):
    """Merge partial attention results with their log-sum-exp.

    ``part_outs``: list of (b, 1, h, d) or (rows, d) fp32 tensors, each normalised
    within its part (e.g. one per sequence shard, from ``fwd_kvcache_int(...,
    out_dtype=torch.float32, return_lse=True)``); ``part_lses``: matching fp32 LSEs.
    The tensors may live on peer GPUs as long as peer access is enabled; the
    result is written on the first tensor's device.
    """
    n = len(part_outs)
    _require(1 <= n <= _lib.BD_MAX_PARTS and len(part_lses) == n, f"need 1..{_lib.BD_MAX_PARTS} parts")
    shape = part_outs[0].shape
    d = shape[-1]
    rows = part_outs[0].numel() // d
    for o, l in zip(part_outs, part_lses):
        _require(o.is_cuda and l.is_cuda and o.dtype == torch.float32 and l.dtype == torch.float32,
                 "partials must be fp32 CUDA tensors")
        _require(o.is_contiguous() and l.is_contiguous() and o.shape == shape and l.numel() == rows,
                 "partials must be contiguous and of equal shape")
    dev = part_outs[0].device
    out = torch.empty(shape, dtype=out_dtype, device=dev)
    lse = torch.empty(part_lses[0].shape, dtype=torch.float32, device=dev) if return_lse else None
    po = (C.c_void_p * n)(*[o.data_ptr() for o in part_outs])
    pl = (C.c_void_p * n)(*[l.data_ptr() for l in part_lses])
    a = _lib.CombineArgs(n_parts=n, part_out=C.cast(po, C.POINTER(C.c_void_p)),
                         part_lse=C.cast(pl, C.POINTER(C.c_void_p)), rows=rows, d=d,
                         out=out.data_ptr(), lse=(lse.data_ptr() if lse is not None else None),
                         out_dtype=_dtype_code(out_dtype))
    with torch.cuda.device(dev):
        _lib.check(_lib.load().bd_combine(C.byref(a), _stream(dev)), "bd_combine")
    return (out, lse) if return_lse else out
