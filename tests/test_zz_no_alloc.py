"""The allocation-free argmax entry point, called through its exported C symbol.

Some users of the library may not allocate device memory when they ask for a greedy token (all memory already
handed to fixed pools, or a C host without any caching allocator). `hb_argmax_noalloc` serves them from a scratch
array built into the library. This test loads the symbol with ctypes, runs it twice in a row (the calls share the
scratch, so the second must not be disturbed by what the first left there) and compares with the regular
two-stage argmax that takes caller-provided scratch and with `torch.argmax`.
"""
import ctypes

import pytest
import torch

from hibana_b200 import _native as nv
from hibana_b200.ops import sampling


def _entry():
    lib = nv.lib()
    fn = lib.hb_argmax_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    fn.restype = ctypes.c_int
    return fn


@pytest.mark.gpu
def test_noalloc_argmax_matches_regular_entry_point_twice():
    fn = _entry()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(11)
    cases = [(torch.randn(64, 151936, generator=g), True), (torch.randn(7, 4099, generator=g).bfloat16(), False)]
    for logits_cpu, is_f32 in cases:
        logits = logits_cpu.to(dev)
        logits[0, 5] = logits[0, 4000] = 99.0                     # tie: lowest index wins in both paths
        want = sampling.argmax(logits)                            # regular entry point (caller-provided scratch)
        for _ in range(2):                                        # two calls in a row share the built-in scratch
            out = torch.full((logits.shape[0],), -1, dtype=torch.int64, device=dev)
            err = ctypes.create_string_buffer(200)
            code = fn(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], int(is_f32),
                      out.data_ptr(), torch.cuda.current_stream().cuda_stream, err, 200)
            torch.cuda.synchronize()
            assert code == 0, err.value
            assert torch.equal(out, want)
            assert torch.equal(out, torch.argmax(logits.float(), dim=-1))     # second oracle: the library argmax
        assert int(want[0]) == 5


@pytest.mark.gpu
def test_noalloc_argmax_refuses_oversized_requests():
    fn = _entry()
    x = torch.zeros(4, 64, device="cuda")
    out = torch.zeros(4, dtype=torch.int64, device="cuda")
    err = ctypes.create_string_buffer(200)
    code = fn(x.data_ptr(), 64, 1025, 64, 1, out.data_ptr(), 0, err, 200)
    assert code == 2 and b"at most 1024 rows" in err.value
    assert fn(None, 64, 4, 64, 1, out.data_ptr(), 0, err, 200) == 1
