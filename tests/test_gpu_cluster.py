"""The cluster form of the split merge (partials exchanged through distributed shared memory)
gives the same attention as the scratch + ticket form and as the oracle."""
import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import encode_cache, kv_values, rel_err, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,hq,hkv,d,seq_len,n_splits,kv_start", [
    ("F8", 32, 8, 128, 8192, 16, 0), ("F8", 32, 8, 128, 1000, 4, 0), ("F8", 64, 8, 128, 5000, 8, 300),
    ("F8", 32, 8, 128, 700, 2, 0), ("F8", 32, 8, 128, 300, 16, 0),       # more splits than 32-row chunks: empty CTAs
    ("F16", 32, 8, 128, 2048, 16, 0), ("F16", 16, 8, 256, 3000, 5, 1976), ("F8", 32, 8, 256, 2000, 3, 0),
])
def test_cluster_merge_matches_oracle_and_ticket_form(ctx, dtype, hq, hkv, d, seq_len, n_splits, kv_start):
    import torch
    odt = {"F16": oracle.F16, "F8": oracle.F8}[dtype]
    rng = np.random.default_rng(seq_len + n_splits)
    frac = 0.01 if dtype == "F8" else 0.0
    k, v = kv_values(rng, (seq_len, hkv, d), frac), kv_values(rng, (seq_len, hkv, d), frac)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, seq_len), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, n_splits=n_splits)
    try:
        for base in range(0, seq_len, 4096):
            n = min(4096, seq_len - base)
            fwd.b_step_kv_write(0, to_dev(k[base:base + n]), to_dev(v[base:base + n]), n, base, 0)
        dq = to_dev(q)
        outs = []
        for on in (False, True):
            ctx.set_cluster_merge(on)
            out = torch.zeros(hq, d, device="cuda")
            for _ in range(2):                      # twice: nothing is left behind by the first call
                fwd.run_flash_attn_split_reduce(dq, out, 0, seq_len - 1, n_splits, 0, kv_start)
            torch.cuda.synchronize()
            ctx.poll()
            outs.append(out.cpu().numpy())
        kc, vc = encode_cache(k, odt), encode_cache(v, odt)
        want = oracle.attention_ref(q, kc, vc, odt, hq, hkv, d, seq_len, kv_start)
        for got in outs:
            if dtype == "F8":
                assert rel_err(got, want) < 3e-2
            else:
                assert float(np.max(np.abs(got - want))) < 2e-3
        assert float(np.max(np.abs(outs[0] - outs[1]))) < 1e-5 * max(1.0, float(np.abs(want).max()))
    finally:
        ctx.set_cluster_merge(False)
        fwd.workspace.destroy()
        cache.destroy()
