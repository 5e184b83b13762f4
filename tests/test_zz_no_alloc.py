"""GPU: the factor-gradient entry point that allocates nothing.

Who needs it: a caller that cannot obtain device memory at the time of the call - a plug-in running
inside another framework's memory plan, a host that owns only the input and output buffers it was
given, or a process whose memory pool is already committed.  For such callers
``b2g_lora_wgrad_static`` keeps the split partials in a fixed 8 MiB array that lives inside the
library image instead of asking for a workspace.

The check: through the C ABI, the new entry point must give exactly the bytes of the existing
``b2g_lora_wgrad`` (same kernels, same summation order, so the tolerance is zero), on two calls in a
row with different inputs (the second call finds the first call's partials still in the array),
and it must refuse a shape whose scratch need is beyond the array.  This file sorts last so that a
run that stops at the first failure has already run every other test; it does not depend on them.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _wgrad_pair(lib_mod, cuda, m, c, r, seed, transpose_out):
    g = torch.Generator(device=cuda).manual_seed(seed)
    s16 = torch.zeros(m, 16, device=cuda, dtype=torch.bfloat16)
    s16[:, :r] = torch.randn(m, r, generator=g, device=cuda).bfloat16()
    t = torch.randn(m, c, generator=g, device=cuda).bfloat16()
    shape = (c, r) if transpose_out else (r, c)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # existing entry point, workspace from the caller
    need = lib_mod.query("b2g_lora_wgrad_workspace_bytes", m, c)
    ws = torch.empty(need // 4, dtype=torch.float32, device=cuda)
    want = torch.empty(shape, device=cuda, dtype=torch.bfloat16)
    lib_mod.call("b2g_lora_wgrad", _ptr(s16), _ptr(t), 2.0, _ptr(want), int(transpose_out), _ptr(ws), need, m, c, r, stream)
    # new entry point: inputs and outputs only
    got = torch.full(shape, float("nan"), device=cuda, dtype=torch.bfloat16)
    lib_mod.call("b2g_lora_wgrad_static", _ptr(s16), _ptr(t), 2.0, _ptr(got), int(transpose_out), m, c, r, stream)
    torch.cuda.synchronize()
    ref = 2.0 * s16[:, :r].float().t() @ t.float()
    return got, want, (ref.t() if transpose_out else ref)


def test_static_scratch_entry_matches_workspace_entry_twice(cuda):
    from b2g import _lib

    assert _lib.query("b2g_lora_wgrad_static_max_bytes") == 8 << 20
    # two calls in a row, different shapes and data: the second starts from the first one's leftovers
    for seed, (m, c, r, tr) in enumerate([(8192, 2048, 16, False), (5000, 512, 4, True)]):
        got, want, ref = _wgrad_pair(_lib, cuda, m, c, r, 100 + seed, tr)
        assert torch.equal(got, want), "the two entry points run the same kernels and must agree bit for bit"
        err = (got.float() - ref).norm() / ref.norm()
        assert float(err) < 1e-2


def test_static_scratch_entry_rejects_oversized_shapes(cuda):
    from b2g import _lib

    m, c = 1 << 12, 1 << 18                                # 16 rank rows x 262144 columns of fp32 partials: 16 MiB
    assert _lib.query("b2g_lora_wgrad_workspace_bytes", m, c) > _lib.query("b2g_lora_wgrad_static_max_bytes")
    dummy = torch.zeros(16, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="needs .* bytes of scratch"):
        _lib.call("b2g_lora_wgrad_static", _ptr(dummy), _ptr(dummy), 1.0, _ptr(dummy), 0, m, c, 16,
                  C.c_void_p(torch.cuda.current_stream().cuda_stream))
