"""rg_b200_attn_decode_static — the flash-decoding entry point for callers that cannot provide scratch memory
(a runtime whose pool owns the GPU's free memory, a serving loop that must avoid cudaMalloc's synchronisation, a
plugin that only receives input and output buffers).  It must give exactly what rg_b200_attn_decode gives, on
repeated calls, because both run the same kernel and differ only in where the split-K scratch lives.  Collected
last on purpose (file name), so a failure here cannot hide the other tests in a stop-at-first-failure run."""
import numpy as np
import pytest
import torch

from refactorgraph_b200 import capi

import _ops as ops

pytestmark = pytest.mark.gpu


def _case(seed, B, nH, nKV, D, lens, dtype=torch.float16):
    rng = np.random.default_rng(seed)
    max_seq = max(lens) + 3
    q = torch.from_numpy(rng.standard_normal((B, nH, D)).astype(np.float32)).to(dtype).cuda()
    kc = torch.from_numpy(rng.standard_normal((B, nKV, max_seq, D)).astype(np.float32)).to(dtype).cuda()
    vc = torch.from_numpy(rng.standard_normal((B, nKV, max_seq, D)).astype(np.float32)).to(dtype).cuda()
    lens_d = torch.tensor(lens, dtype=torch.int64, device="cuda")
    return q, kc, vc, lens_d, ops.kv_layout(nKV, D, max_seq), max(lens)


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    stream = torch.cuda.current_stream().cuda_stream
    for seed, shape in enumerate([(2, 8, 2, 128, [1500, 777]), (1, 32, 32, 128, [2049])]):
        q, kc, vc, lens_d, kv, max_len = _case(seed, *shape)
        want, _ = ops.attn_decode(q, kc, vc, lens_d, kv, max_len)
        p = capi.AttnDecodeParams(ops.DT[q.dtype], q.shape[0], q.shape[1], max_len, kv)
        assert capi.workspace("attn_decode", p) <= capi.load().rg_b200_attn_decode_static_capacity()
        for _ in range(2):  # the second call finds the array as the first one left it
            got = torch.full_like(q, float("nan"))
            capi.attn_decode_static(p, [q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens_d.data_ptr(), 0], [got.data_ptr()], stream=stream)
            torch.cuda.synchronize()
            assert torch.equal(got, want)


def test_static_scratch_rejects_requests_beyond_its_capacity():
    # 1024 sequences x 128 heads with a 16k context need far more partial records than the fixed array holds
    kv = ops.kv_layout(8, 128, 16384)
    p = capi.AttnDecodeParams(capi.FP16, 1024, 128, 16384, kv)
    assert capi.workspace("attn_decode", p) > capi.load().rg_b200_attn_decode_static_capacity()
    assert capi.attn_decode_static(p, [1, 1, 1, 1, 0], [1], check=False) == capi.ERR_LIMIT


def test_static_scratch_limit_follows_the_kernel_that_will_run():
    # Grouped-query shapes use a different record size than the general kernel.  In the window where only the
    # grouped-query layout exceeds the array, the call must be refused (return code only: nothing is launched).
    lib = capi.load()
    cap = lib.rg_b200_attn_decode_static_capacity()
    refused = fits = 0
    for batch in range(470, 520, 2):
        p = capi.AttnDecodeParams(capi.FP16, batch, 32, 1024, ops.kv_layout(4, 128, 1024))
        need = capi.workspace("attn_decode", p)
        if need > cap:
            assert capi.attn_decode_static(p, [1, 1, 1, 1, 0], [1], check=False) == capi.ERR_LIMIT, (batch, need)
            refused += 1
        else:
            fits += 1
    assert refused and fits, "the sweep should straddle the capacity"
    # a grouped-query case just below the limit runs, and matches the workspace entry point
    q, kc, vc, lens_d, kv, max_len = _case(7, 24, 32, 4, 128, [40 + 3 * i for i in range(24)])
    want, _ = ops.attn_decode(q, kc, vc, lens_d, kv, max_len)
    p = capi.AttnDecodeParams(ops.DT[q.dtype], q.shape[0], q.shape[1], max_len, kv)
    got = torch.full_like(q, float("nan"))
    capi.attn_decode_static(p, [q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens_d.data_ptr(), 0], [got.data_ptr()],
                            stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
