"""cats_mlp_static: the entry point for callers that cannot allocate device memory.

Some users of this library only ever get buffers handed to them (a plugin inside a host
application, a runtime with a fixed memory budget) and cannot call cudaMalloc for a workspace.
``cats_mlp_static`` serves them with a scratch array that is compiled into the library.  This
test drives it through the C ABI exactly as such a caller would - raw pointers, no workspace -
and checks it against ``cats_mlp`` (caller-provided workspace) on two calls in a row, the second
with different inputs, because the built-in array is shared and keeps the previous call's
contents.  The file is named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm())


@pytest.mark.parametrize("dt,code,tol", [(torch.float16, 1, 2e-3), (torch.float32, 0, 1e-5),
                                          (torch.bfloat16, 2, 1e-2)])
def test_static_entry_point_matches_cats_mlp_twice(dt, code, tol, cuda_device):
    from cats_b200 import _lib, ops, synth

    L = _lib.lib()
    H, I, B = 1024, 2752, 2
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    for call, seed in enumerate((3, 4)):
        layer = synth.make_layer(H, I, dt, cuda_device, seed, sparsity=0.5, std=0.04)
        x = synth.make_x(B, H, dt, cuda_device, 100 + seed)
        ref = ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold)      # existing entry point
        out = torch.full_like(x, float("nan"))
        st = L.cats_mlp_static(x.data_ptr(), layer.wg.data_ptr(), layer.wu.data_ptr(),
                               layer.wdt.data_ptr(), B, H, I, code, float(layer.threshold),
                               out.data_ptr(), stream)
        assert st == 0, L.cats_status_string(st).decode()
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        assert rel_l2(out, ref) <= tol, f"call {call}: {rel_l2(out, ref):.2e}"


def test_static_entry_point_refuses_shapes_beyond_its_array(cuda_device):
    from cats_b200 import _lib

    L = _lib.lib()
    limit = L.cats_mlp_static_limit()
    assert limit == 8 << 20
    assert L.cats_workspace_bytes(1, 8192, 28672) <= limit       # the largest documented shape fits
    H, I = 8192, 131072                                           # needs ~18 MiB of scratch
    assert L.cats_workspace_bytes(1, H, I) > limit
    x = torch.zeros(16, device=cuda_device, dtype=torch.float16)  # never touched: refused first
    p = x.data_ptr()
    st = L.cats_mlp_static(p, p, p, p, 1, H, I, 1, 0.1, p, None)
    assert st == -8
    assert "cats_mlp_static" in L.cats_status_string(st).decode()
