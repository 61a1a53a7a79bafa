"""GPU: the allocation-free variant of the step against the regular entry point.

Some users of this library cannot let it allocate device memory: the card may be fully owned by
another allocator, or the call sits on a path where allocations are forbidden. For them
`gefen_b200_automatic_gefen_fused_update_from_vmean_static_ws` keeps the codebook tables in an array
that is part of the library image. This test drives both entry points through the C ABI on the same
inputs, twice in a row (the second call re-uses the array the first one filled, with a different
codebook), and asks for identical outputs. It is collected last on purpose, and it makes no
assumption about what ran before it.
"""
import ctypes

import pytest
import torch

from tests.util import make_grad, make_param, reference_like_codebook

pytestmark = pytest.mark.gpu


def _call(lib, fn_static, tensors, cb, ws, args, stream, dtype_tag):
    p, g, codes, mag, v = tensors
    nb, period = g.shape
    common_head = (p.data_ptr(), g.data_ptr(), dtype_tag, codes.data_ptr(), mag.data_ptr(), dtype_tag, v.data_ptr(),
                   dtype_tag, cb.data_ptr(), cb.numel())
    tail = (0, nb, period) + args + (stream,)
    if fn_static:
        return lib.gefen_b200_automatic_gefen_fused_update_from_vmean_static_ws(*common_head, *tail)
    return lib.gefen_b200_automatic_gefen_fused_update_from_vmean(*common_head, ws.data_ptr(), *tail)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_workspace_step_matches_regular_step(cuda_device, dtype):
    from gefen_b200 import _lib

    lib = _lib.load()
    tag = _lib.dtype_tag(dtype)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    args = (0.9, 3e-4, 1 - 0.9 ** 2, 1 - 0.999 ** 2, 1e-8)
    books = [reference_like_codebook(seed=1).to(cuda_device), reference_like_codebook(seed=2, k=64).to(cuda_device)]
    for nb, period in [(48, 2048), (100, 24)]:          # the staged vector kernel and the generic one
        base = [make_param((nb, period), 3, 0, dtype), make_grad((nb, period), 3, 0, 0, dtype),
                torch.randint(0, 64, (nb, period), dtype=torch.uint8),
                (torch.rand(nb, 1) * 2e-3).to(dtype), (torch.rand(nb, 1) * 1e-6 + 1e-9).to(dtype)]
        regular = [t.clone().to(cuda_device) for t in base]
        static = [t.clone().to(cuda_device) for t in base]
        for cb in books:                                 # two calls in a row, the array is re-used
            ws = _lib.codebook_workspace(cb)
            _lib.check(_call(lib, False, regular, cb, ws, args, stream, tag))
            _lib.check(_call(lib, True, static, cb, None, args, stream, tag))
            torch.cuda.synchronize()
            for a, b in zip(regular, static):
                assert torch.equal(a, b)


def test_static_workspace_step_rejects_oversized_codebook(cuda_device):
    from gefen_b200 import _lib

    lib = _lib.load()
    cb = torch.linspace(-1, 1, 300, device=cuda_device)
    t = [torch.zeros(8, 64, device=cuda_device), torch.zeros(8, 64, device=cuda_device),
         torch.zeros(8, 64, dtype=torch.uint8, device=cuda_device), torch.zeros(8, 1, device=cuda_device),
         torch.zeros(8, 1, device=cuda_device)]
    with pytest.raises(ValueError, match="at most 256"):
        _lib.check(_call(lib, True, t, cb, None, (0.9, 1e-3, 0.1, 0.001, 1e-8), None, _lib.F32))
