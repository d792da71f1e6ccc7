# SPDX-License-Identifier: MIT
"""`bl_argmax_noalloc`: the arg max entry point for callers that may not
allocate device memory (allocator callbacks, fixed memory budgets).  It is
called here the way such a caller would call it -- through the exported C symbol of the library, with raw pointers -- and must
agree with the regular entry point (`_C.argmax`, which takes its scratch from
the caller) on two calls in a row, since both calls share one built-in scratch
array.  The file name sorts last so that a run that stops at the first failure
has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import barlink_sm86_b200 as bl

    ext = bl.load_extension()
    lib = ctypes.CDLL(ext.__file__)
    fn = lib.bl_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return ext, fn


def _call(fn, logits, offset, with_val=True):
    rows, n = logits.shape
    idx = torch.full((rows,), -1, dtype=torch.int32, device=logits.device)
    val = torch.zeros(rows, dtype=torch.float32, device=logits.device)
    err = ctypes.create_string_buffer(512)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(logits.data_ptr(), rows, n, logits.stride(0), offset, idx.data_ptr(),
            val.data_ptr() if with_val else None, ctypes.c_void_p(stream), err, 512)
    return rc, err.value.decode(), idx, val


def test_no_alloc_argmax_matches_regular_entry_point_twice():
    ext, fn = _lib()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different shapes back to back: the second call reuses the scratch
    # array that still holds the first call's partial results
    for rows, n, offset in ((64, 152064, 0), (5, 19008, 7)):
        logits = torch.randn(rows, n, device="cuda", generator=g).to(torch.bfloat16)
        logits[rows // 2, 3] = logits[rows // 2, n - 2] = 99.0  # tie: the lower index wins
        want_idx, want_val = ext.argmax(logits, offset)
        rc, msg, idx, val = _call(fn, logits, offset)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.equal(idx, want_idx)
        assert torch.equal(val, want_val)
        assert int(idx[rows // 2]) == 3 + offset


def test_no_alloc_argmax_against_a_plain_pytorch_oracle_with_row_pitch_and_without_values():
    """Rows that are views into a wider buffer (row pitch larger than the row length) and a caller
    that does not want the maxima (val = NULL), checked against torch.max directly, twice."""
    _, fn = _lib()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(12)
    for rows, n, pitch, offset in ((33, 19000, 19008, 5), (7, 1000, 4096, 0)):
        wide = torch.randn(rows, pitch, device="cuda", generator=g).to(torch.bfloat16)
        wide[:, n:] = 1000.0   # beyond the row: must not be looked at
        logits = wide[:, :n]
        assert logits.stride(0) == pitch > n
        want_val, want_idx = logits.float().max(dim=1)
        # lowest index on ties
        cols = torch.arange(n, device="cuda")[None, :].expand(rows, n)
        first = torch.where(logits.float() == want_val[:, None], cols, torch.full_like(cols, n)).min(dim=1).values
        for with_val in (True, False):
            rc, msg, idx, val = _call(fn, logits, offset, with_val)
            assert rc == 0, msg
            torch.cuda.synchronize()
            assert torch.equal(idx.long(), first + offset)
            if with_val:
                assert torch.equal(val, want_val)
            else:
                assert torch.all(val == 0)   # untouched


def test_no_alloc_argmax_rejects_too_many_rows():
    _, fn = _lib()
    logits = torch.zeros(4097, 8, dtype=torch.bfloat16, device="cuda")
    rc, msg, idx, _ = _call(fn, logits, 0)
    assert rc == -1
    assert "4096" in msg
    torch.cuda.synchronize()
    assert torch.all(idx == -1)  # nothing ran
