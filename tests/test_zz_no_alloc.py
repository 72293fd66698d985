"""The allocation-free attention entry point, for hosts that may not call cudaMalloc while
running (all device memory carved out at start-up, or a thread that cannot take cudaMalloc's
device-wide synchronisation).  Its split-K scratch is a fixed device array inside the library,
so the check is: same results as the workspace-based entry point, on two calls in a row that
reuse (and must not be confused by) whatever the previous call left in that array.

Collected last on purpose: a run that stops at the first failure has by then run everything else.
"""
import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import kv_values, to_dev

pytestmark = pytest.mark.gpu

ABS_TOL = 1e-3      # the tolerance of the attention tests for F32 / F16 caches
FP8_REL_TOL = 3e-2  # relative to the output's max, FP8 cache


def _run_both(ctx, ws, dtype, hq, hkv, d, L, start, n_splits, softcap, seed):
    import torch
    L_ = ctx._lib
    rng = np.random.default_rng(seed)
    fp8 = dtype == oracle.F8
    k = oracle.store(kv_values(rng, (L + 5, hkv, d), outlier_frac=0.01 if fp8 else 0.0), dtype)
    v = oracle.store(kv_values(rng, (L + 5, hkv, d), outlier_frac=0.01 if fp8 else 0.0), dtype)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    dq, dk, dv = to_dev(q), to_dev(k), to_dev(v)
    scale = float(1.0 / np.sqrt(d))
    a = torch.full((hq, d), float("nan"), device="cuda")
    b = torch.full((hq, d), float("nan"), device="cuda")
    ctx.check(L_.vfkv_flash_attn_split_reduce(ctx.handle, ws.handle, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                              a.data_ptr(), dtype, hq, hkv, d, L, L + 5, scale, start, softcap,
                                              n_splits, None))
    rc = L_.vfkv_flash_attn_split_reduce_noalloc(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), b.data_ptr(), dtype,
                                                 hq, hkv, d, L, L + 5, scale, start, softcap, n_splits, None)
    assert rc == 0, L_.vfkv_noalloc_last_error()
    torch.cuda.synchronize()
    a, b = a.cpu().numpy(), b.cpu().numpy()
    want = oracle.attention_ref(q, k.reshape(L + 5, hkv, d), v.reshape(L + 5, hkv, d), dtype, hq, hkv, d, L, start,
                                scale, softcap)
    assert np.isfinite(b).all()
    if fp8:
        m = float(np.max(np.abs(want)))
        assert float(np.max(np.abs(b - a))) < FP8_REL_TOL * m and float(np.max(np.abs(b - want))) < FP8_REL_TOL * m
    else:
        assert float(np.max(np.abs(b - a))) < ABS_TOL and float(np.max(np.abs(b - want))) < ABS_TOL


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row(ctx):
    L_ = ctx._lib
    assert L_.vfkv_noalloc_scratch_bytes() == 256 + 4 * 512 * 1024
    ws = vf.Workspace(ctx, 1, 64, 256, 64)
    try:
        # first call: many splits, so the scratch is left full of this problem's partials
        _run_both(ctx, ws, oracle.F8, 32, 8, 128, 3000, 0, 16, 0.0, seed=1)
        # second call straight after: other shape, dtype, window, soft-cap and split count
        _run_both(ctx, ws, oracle.F16, 16, 8, 256, 700, 150, 5, 30.0, seed=2)
        # and a single-split call, which bypasses the scratch altogether
        _run_both(ctx, ws, oracle.F32, 64, 8, 128, 90, 0, 0, 0.0, seed=3)
    finally:
        ws.destroy()


def test_noalloc_entry_rejects_what_does_not_fit(ctx):
    import torch
    L_ = ctx._lib
    x = torch.zeros(64 * 512, device="cuda")
    p = x.data_ptr()
    E_UNSUP, E_INVAL = vf.kv_cache.ERR_UNSUPPORTED, vf.kv_cache.ERR_INVALID
    # 64 heads x 64 splits x (256 + 2) floats = 1 056 768 > 524 288
    assert L_.vfkv_flash_attn_split_reduce_noalloc(p, p, p, p, oracle.F16, 64, 8, 256, 64, 64, 1.0, 0, 0.0, 64,
                                                   None) == E_UNSUP
    assert b"exceeds the built-in scratch" in L_.vfkv_noalloc_last_error()
    assert L_.vfkv_flash_attn_split_reduce_noalloc(p, p, p, p, oracle.F16, 64, 8, 96, 8, 8, 1.0, 0, 0.0, 1,
                                                   None) == E_UNSUP
    assert L_.vfkv_flash_attn_split_reduce_noalloc(None, p, p, p, oracle.F16, 64, 8, 128, 8, 8, 1.0, 0, 0.0, 1,
                                                   None) == E_INVAL
    assert L_.vfkv_flash_attn_split_reduce_noalloc(p, p, p, p, oracle.F16, 64, 8, 128, 9, 8, 1.0, 0, 0.0, 1,
                                                   None) == E_INVAL
    assert L_.vfkv_flash_attn_split_reduce_noalloc(p, p, p, p, 7, 64, 8, 128, 8, 8, 1.0, 0, 0.0, 1, None) == E_INVAL
    torch.cuda.synchronize()


def test_noalloc_entry_leaves_the_free_device_memory_unchanged(ctx):
    """What the entry point is for: once a kernel shape has been used (the driver loads a kernel's
    code when it is first launched), further calls take no device memory at all.  Free memory as
    the driver reports it is read before and after a series of calls, head_dim 512 included (that
    shape configures its kernel's dynamic shared memory on the way in)."""
    import torch
    L_ = ctx._lib
    rng = np.random.default_rng(9)
    cases = []
    for dtype, hq, hkv, d, L, n_splits in ((oracle.F8, 32, 8, 128, 2000, 8), (oracle.F16, 16, 8, 256, 600, 4),
                                            (oracle.F32, 8, 2, 512, 300, 3), (oracle.F32, 8, 2, 64, 100, 1)):
        k = oracle.store(kv_values(rng, (L, hkv, d), outlier_frac=0.0), dtype)
        q = rng.standard_normal((hq, d), dtype=np.float32)
        out = torch.zeros(hq, d, device="cuda")
        cases.append((to_dev(q), to_dev(k), out, dtype, hq, hkv, d, L, n_splits))

    def call_all():
        for dq, dk, out, dtype, hq, hkv, d, L, n_splits in cases:
            rc = L_.vfkv_flash_attn_split_reduce_noalloc(dq.data_ptr(), dk.data_ptr(), dk.data_ptr(), out.data_ptr(),
                                                         dtype, hq, hkv, d, L, L, float(1.0 / np.sqrt(d)), 0, 0.0,
                                                         n_splits, None)
            assert rc == 0, L_.vfkv_noalloc_last_error()

    call_all()                                      # first use of every kernel shape
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        call_all()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    for _, _, out, *_ in cases:
        assert bool(torch.isfinite(out).all())
