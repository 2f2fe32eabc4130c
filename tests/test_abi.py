"""CPU: the C-ABI library loads, exports what include/bitdecode.h declares, validates
arguments before touching a device, and its host-side planning arithmetic is sound."""
import ctypes as C
import os
import random
import re

import numpy as np
import pytest

from bitladder_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "bitdecode.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bd_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.load()
    names = _declared_functions()
    assert {"bd_pack", "bd_decode", "bd_combine", "bd_decode_workspace_bytes", "bd_plan_splits"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/bitdecode.h but not exported"
    assert set(_lib.EXPORTS) == set(names)


def test_version_and_error_strings():
    lib = _lib.load()
    assert lib.bd_version() >= 201
    for code in range(0, -12, -1):
        assert len(_lib.strerror(code)) > 1
    assert "unknown" in _lib.strerror(-99)


def test_struct_sizes_match_the_header_layout():
    # pointers and int64 first, then int32 fields: no padding surprises between ctypes and the C structs
    assert C.sizeof(_lib.PackArgs) == 2 * 8 + 6 * 8 + 4 * 8 + 6 * 8 + 9 * 4 + 4      # nine int32 fields, padded to 8
    assert C.sizeof(_lib.DecodeArgs) % 8 == 0
    assert _lib.DecodeArgs.workspace_bytes.offset == C.sizeof(_lib.DecodeArgs) - 56
    assert _lib.DecodeArgs.advance.offset == C.sizeof(_lib.DecodeArgs) - 48        # three int32 and padding, then the rotary fields
    assert _lib.DecodeArgs.test_starve.offset == C.sizeof(_lib.DecodeArgs) - 40


def test_argument_validation_needs_no_device():
    lib = _lib.load()
    assert lib.bd_pack(None, None) == -1
    assert lib.bd_decode(None, None) == -1
    a = _lib.PackArgs()
    assert lib.bd_pack(C.byref(a), None) == -1                     # null pointers
    buf = (C.c_char * 64)()
    ptr = C.addressof(buf)
    a = _lib.PackArgs(k=ptr, v=ptr, k_pack=ptr, k_params=ptr, v_pack=ptr, v_params=ptr,
                      b=1, s=128, h_k=1, d=128, bits=3, group=128, dtype=0)
    assert lib.bd_pack(C.byref(a), None) == -2                     # bits = 3
    a.bits, a.d = 4, 64
    assert lib.bd_pack(C.byref(a), None) == -2                     # head dim 64
    a.d, a.s = 128, 100
    assert lib.bd_pack(C.byref(a), None) == -1                     # not whole pack blocks
    d = _lib.DecodeArgs(q=ptr, out=ptr, k_pack=ptr, k_params=ptr, v_pack=ptr, v_params=ptr,
                        b=1, h=34, h_k=8, d=128, s=128, s_cap=128, bits=4, group=128)
    assert lib.bd_decode(C.byref(d), None) == -1                   # heads do not divide
    d.h = 8 * 17
    assert lib.bd_decode(C.byref(d), None) == -2                   # more than 16 query heads per KV head
    d.h, d.group = 32, 16
    assert lib.bd_decode(C.byref(d), None) == -2                   # group 16 not built
    c = _lib.CombineArgs(n_parts=0)
    assert lib.bd_combine(C.byref(c), None) == -1


def test_plan_splits_fills_the_machine():
    lib = _lib.load()
    plan = lambda b, hk, s, bits=4, sm=148, c=3: lib.bd_plan_splits(b, hk, s, bits, sm, c)
    assert plan(8, 8, 32768) == 55                    # 55 rows x 8 heads = 440 CTAs <= 444 resident
    assert plan(32, 32, 16384) == 13
    assert plan(16, 1, 131072) == 444
    assert plan(1, 8, 4096) == 16                     # small problem: two blocks per range
    assert plan(2, 8, 4096) == 32
    assert plan(8, 8, 32768, c=0) == 18               # the kernel's own residency: one CTA per SM
    assert plan(1, 8, 128) == 1
    assert plan(1, 1024, 4096) == 1                   # more heads than slots: one row
    assert plan(8, 8, 32768, 2) == 55


def _segments(lib, table, b, n, R, row):
    out = np.zeros(4 * 4096, np.int32)
    k = lib.bd_partition_segments(None if table is None else table.ctypes.data, b, n, R, row, out.ctypes.data, 4096)
    assert k >= 0
    return out[:4 * k].reshape(k, 4)


def _parts(lib, table, b, n, R, ib):
    out = np.zeros(4096, np.int32)
    k = lib.bd_partition_parts(None if table is None else table.ctypes.data, b, n, R, ib, out.ctypes.data, 4096)
    assert k >= 0
    return list(out[:k])


def test_partition_covers_every_unit_once_and_is_balanced():
    """The arithmetic the decode kernel and its merge share: every unit (pack block or tail
    chunk) belongs to exactly one row, rows differ by at most one unit, partial slots (row +
    sequence) never clash, every sequence without units has exactly one row that answers for it,
    and the merge finds exactly the rows that wrote.  The kernel cuts twice with the same
    arithmetic (CTAs, then warps inside a CTA): the finer cut must nest inside the coarser."""
    lib = _lib.load()
    rnd = random.Random(7)
    for _ in range(600):
        b, R = rnd.randint(1, 12), rnd.randint(1, 40)
        if rnd.random() < 0.3:
            n, table, counts = rnd.randint(0, 20), None, None
            counts = [n] * b
        else:
            counts = [rnd.choice([0, 0, 1, 2, 3, 5, 17, rnd.randint(0, 40)]) for _ in range(b)]
            firsts = np.cumsum([0] + counts)
            table = np.zeros(2 * (b + 1), np.int32)
            table[0:2 * b:2], table[1:2 * b:2], table[2 * b], n = firsts[:-1], counts, firsts[-1], 0
        cover, empties, slots = {}, {}, set()
        rows_of = {ib: [] for ib in range(b)}
        per_row = []
        for row in range(R):
            tot = 0
            for ib, u0, u1, owns in _segments(lib, table, b, n, R, row):
                if u1 > u0:
                    assert not owns
                    assert (row + ib) not in slots
                    slots.add(row + ib)
                    rows_of[ib].append(row)
                    tot += u1 - u0
                    for u in range(u0, u1):
                        assert (ib, u) not in cover
                        cover[(ib, u)] = row
                else:
                    assert owns and counts[ib] == 0
                    assert ib not in empties
                    empties[ib] = row
            per_row.append(tot)
        assert len(cover) == sum(counts)
        assert set(empties) == {ib for ib in range(b) if counts[ib] == 0}
        assert max(per_row) - min(per_row) <= 1
        for ib in range(b):
            assert _parts(lib, table, b, n, R, ib) == rows_of[ib]
        # the warp-level cut (W rows per CTA row) nests inside the CTA-level cut
        W = rnd.choice([2, 8, 12])
        for row in range(R):
            coarse = [(ib, u) for ib, u0, u1, _ in _segments(lib, table, b, n, R, row) for u in range(u0, u1)]
            fine = [(ib, u) for w in range(W) for ib, u0, u1, _ in _segments(lib, table, b, n, R * W, row * W + w)
                    for u in range(u0, u1)]
            assert fine == coarse
