"""cats_mlp_static: the entry point for callers that cannot allocate device memory.

Some users of this library only ever get buffers handed to them (a plugin inside a host
application, a runtime with a fixed memory budget) and cannot call cudaMalloc for a workspace.
``cats_mlp_static`` serves them with a scratch array that is compiled into the library.  This
test drives it through the C ABI exactly as such a caller would - raw pointers, no workspace -
and checks it against ``cats_mlp`` (caller-provided workspace) and the CPU oracle on several
calls in a row with changing shapes and batch sizes, because the built-in array is shared and
keeps the previous call's contents.  The file is named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm())


@pytest.mark.parametrize("dt,code,tol", [(torch.float16, 1, 1e-2), (torch.float32, 0, 1e-5),
                                          (torch.bfloat16, 2, 1e-2)])
def test_static_entry_point_matches_cats_mlp_and_the_oracle_on_changing_shapes(dt, code, tol,
                                                                               cuda_device):
    """Calls in a row with DIFFERENT (H, I, B): the built-in array is shared and keeps what the
    previous call left, and where the accumulators and lists sit in it depends on H and I, so a
    clear that is missing shows up exactly when the shape changes (a large batch followed by a
    small one, a wide layer followed by a narrow one).  Every call is checked against the CPU
    oracle and against cats_mlp with a caller workspace."""
    from cats_b200 import _lib, ops, synth
    from oracle import cats_oracle as O

    L = _lib.lib()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    to_np = lambda t: t.detach().float().cpu().numpy()
    for call, (H, I, B, seed) in enumerate([(2048, 4096, 4, 3), (1024, 2752, 1, 4),
                                            (1024, 2752, 2, 5), (2048, 4096, 1, 6)]):
        layer = synth.make_layer(H, I, dt, cuda_device, seed, sparsity=0.5)
        x = synth.make_x(B, H, dt, cuda_device, 100 + seed)
        ref = ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold)      # existing entry point
        out = torch.full_like(x, float("nan"))
        st = L.cats_mlp_static(x.data_ptr(), layer.wg.data_ptr(), layer.wu.data_ptr(),
                               layer.wdt.data_ptr(), B, H, I, code, float(layer.threshold),
                               out.data_ptr(), stream)
        assert st == 0, L.cats_status_string(st).decode()
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        assert rel_l2(out, ref) <= tol, f"call {call}: {rel_l2(out, ref):.2e} vs cats_mlp"
        # the oracle on the same (rounded) inputs, with the kernel's own mask where a gate value
        # sits within the 1e-3 band of the threshold
        flag = torch.zeros((B, I), dtype=torch.bool, device=cuda_device)
        ops.gate(x, layer.wg, layer.threshold, flag_dense=flag)
        xn = to_np(x).reshape(B, H)
        ref64 = O.dense_masked_mlp(xn, to_np(layer.wg), to_np(layer.wu), to_np(layer.wdt).T,
                                   layer.threshold, dtype=np.float64)
        flips, outside = O.mask_band_check(ref64["post_act"], flag.cpu().numpy(), layer.threshold)
        assert outside == 0
        exp = O.dense_masked_mlp(xn, to_np(layer.wg), to_np(layer.wu), to_np(layer.wdt).T,
                                 layer.threshold, mask=flag.cpu().numpy() if flips else None)
        err = O.rel_l2(to_np(out).reshape(B, H), exp["out"])
        assert err <= tol, f"call {call} ({H}x{I}, B={B}): rel L2 {err:.2e} vs the oracle"
    status = _lib.ctypes.c_int(-1)
    assert L.cats_mlp_static_status(_lib.ctypes.byref(status), stream) == 0
    assert status.value == 0


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
