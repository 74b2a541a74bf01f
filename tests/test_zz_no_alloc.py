"""The decode-attention entry point that allocates nothing (rl_attention_decode_static),
called through its exported C symbol and compared with the entry point that takes
caller-allocated scratch.  Collected last on purpose: a run that stops at the first
failure has then already run every other test."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_entry():
    from rustyllm_b200 import kernels
    lib = kernels.library()
    fn = lib.rl_attention_decode_static
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.restype = i
    fn.argtypes = [p, i, p, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p]
    return kernels, lib, fn


def _call_static(fn, lib, q, kp, vp, pt, slots, kv_lens, out, H, G, hd, splits):
    rc = fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vp.data_ptr(), pt.data_ptr(), pt.shape[1],
            slots.data_ptr(), kv_lens.data_ptr(), out.data_ptr(), out.stride(0), q.shape[0], H, G, hd,
            1.0 / math.sqrt(hd), 0, splits, torch.cuda.current_stream().cuda_stream)
    return rc, lib.rl_last_error().decode()


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from test_kernels_gpu import _attention_case, _decode_inputs, _tol
    kernels, lib, fn = _static_entry()
    # two different calls back to back: the second finds the first one's partial results
    # in the shared scratch and must not be disturbed by them
    for H, G, hd, lens, splits, seed in [(32, 8, 128, [700, 33, 1, 257], 7, 1),
                                         (6, 2, 64, [90, 513], 5, 2)]:
        q, kp, vp, pt, slots, kv_lens, _ = _decode_inputs(
            _attention_case(torch.bfloat16, H, G, hd, [1] * len(lens), lens, seed=seed))
        want = torch.empty(len(lens), H * hd, dtype=torch.bfloat16, device=DEV)
        kernels.attention_decode(q, kp, vp, pt, slots, kv_lens, want, H, G, hd, 1.0 / math.sqrt(hd), num_splits=splits)
        got = torch.full_like(want, float("nan"))
        rc, msg = _call_static(fn, lib, q, kp, vp, pt, slots, kv_lens, got, H, G, hd, splits)
        assert rc == 0, msg
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), **_tol(torch.bfloat16))


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from test_kernels_gpu import _attention_case, _decode_inputs
    kernels, lib, fn = _static_entry()
    H, G, hd = 32, 8, 128
    lens = [20] * 9
    q, kp, vp, pt, slots, kv_lens, _ = _decode_inputs(_attention_case(torch.bfloat16, H, G, hd, [1] * 9, lens, seed=3))
    out = torch.zeros(9, H * hd, dtype=torch.bfloat16, device=DEV)
    # 9 x 32 x 32 x 130 = 1,198,080 floats > 2^20
    rc, msg = _call_static(fn, lib, q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 32)
    assert rc != 0 and "exceed the built-in" in msg
    assert torch.count_nonzero(out).item() == 0          # nothing was launched
    rc, msg = _call_static(fn, lib, q, kp, vp, pt, slots, kv_lens, out, H, G, hd, 1)   # one split needs no scratch
    assert rc == 0, msg
