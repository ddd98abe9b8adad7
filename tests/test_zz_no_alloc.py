"""The allocation-free BitLinear entry point against the regular one.

Kept in a file of its own that sorts last, so that a run which stops at the first failure has
already run every other test.  The entry point serves callers that may not allocate device
memory when they run the operator (inside someone else's captured graph, under a fixed
memory budget, in a loop that forbids driver allocations); its scratch is a fixed array in
the library, so two calls in a row must both be right without anything being reset by hand.
"""
import numpy as np
import pytest
import torch

from oracle import np_oracle as O

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n,k,m", [(2560, 2560, 1), (3840, 2560, 4), (13824, 2560, 8), (2560, 6912, 3)])
def test_noalloc_entry_matches_regular_entry_twice(n, k, m):
    from bitnet_b200 import _lib, ops, pack_weight

    L = _lib.lib
    q, _ = O.synth_weights(n, k, seed=n + m)
    weight = pack_weight.convert_weight_int8_to_int2(_dev(q))
    ws = torch.tensor([0.5, 1.25, 0.875, 2.0, 0.75, 1.5], dtype=torch.bfloat16, device="cuda")
    for call in range(2):                                   # the array keeps the previous call's state
        y, a, _ = O.act_quant(O.synth_acts(m, k, seed=100 * call + k))
        y_d = _dev(y)
        s = _dev(O.to_bf16(a)).bfloat16()
        want = ops.bitnet_int8xint2_linear(y_d, weight, s, ws)          # regular entry point
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        st = L.bitlinear_int8xint2_noalloc(_lib.ptr(y_d), _lib.ptr(weight), _lib.ptr(got), _lib.ptr(s), _lib.ptr(ws),
                                           m, n, k, _lib.stream_ptr())
        assert st == 0, L.bitnet_status_string(st)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))   # same kernel arithmetic: bit-equal
        # and right in absolute terms
        seg = O.ref_gpu_scale_segments(n, k)
        ref = O.to_bf16(O.rescale(O.matmul_i32(y, q), O.to_bf16(a), ws.float().cpu().numpy()[: len(seg)], seg))
        assert np.array_equal(got.float().cpu().numpy(), ref)


def test_noalloc_entry_rejects_what_the_fixed_array_cannot_hold():
    from bitnet_b200 import _lib

    L = _lib.lib
    t = torch.zeros(1 << 16, dtype=torch.int8, device="cuda")
    b = torch.zeros(1 << 16, dtype=torch.bfloat16, device="cuda")
    args = (_lib.ptr(t), _lib.ptr(t), _lib.ptr(b), _lib.ptr(b), _lib.ptr(b))
    assert L.bitlinear_int8xint2_noalloc(*args, 9, 256, 128, None) == 4        # too many tokens
    assert L.bitlinear_int8xint2_noalloc(*args, 1, 16384 + 16, 128, None) == 4  # too many rows
    assert L.bitlinear_int8xint2_noalloc(*args, 1, 250, 128, None) == 2         # not a multiple of 16
    assert L.bitlinear_int8xint2_noalloc(*args, 1, 256, 100, None) == 2
    assert L.bitlinear_int8xint2_noalloc(None, *args[1:], 1, 256, 128, None) == 1
    assert L.bitnet_status_string(4) == b"size exceeds a fixed capacity"
    torch.cuda.synchronize()
    assert not b.any()                                                        # nothing was written
