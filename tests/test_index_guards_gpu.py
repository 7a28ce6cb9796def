"""Device-read indices are never trusted.  A generation loop advances positions, lengths and tokens on the GPU, so a
kernel may be handed a position past the end of the cache, a length beyond what the launch was sized for, a token id
outside the vocabulary or a block-table entry outside the cache.  Every such case must: leave memory it does not own
untouched (checked with whole-buffer comparisons and guard regions), set bit 5 of rg_b200_error_state, fault nothing,
and leave the kernel's workspace usable for the next, valid call.  The out-of-range values are chosen on the host; no
case here is expected to fault, trap or hang."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi

import _ops as ops

pytestmark = pytest.mark.gpu
INDEX_BIT = 32
GUARD = 4096   # elements of guard pattern after each buffer


def _guarded(shape, dtype=torch.float16, fill=None):
    """A tensor followed by a guard region inside the same allocation; returns (view, whole buffer, guard slice)."""
    n = int(np.prod(shape))
    buf = torch.full((n + GUARD,), 7.0, dtype=dtype, device="cuda")
    view = buf[:n].view(*shape)
    if fill is None:
        view.normal_()
    else:
        view.fill_(fill)
    return view, buf, buf[n:]


def _expect_index_error_then_clear():
    lib = capi.load()
    st = lib.rg_b200_error_state()
    assert st >= 0 and st & INDEX_BIT, f"error state {st}: the out-of-range index was not reported"
    assert (st & ~INDEX_BIT) == 0, f"error state {st}: an unrelated error bit is set"
    assert lib.rg_b200_error_clear() == capi.OK
    assert lib.rg_b200_error_state() == 0


@pytest.fixture(autouse=True)
def _clean_error_state():
    lib = capi.load()
    assert lib.rg_b200_error_state() == 0, "an earlier test left an error behind"
    yield
    lib.rg_b200_error_clear()


@pytest.mark.parametrize("tokens", [2, 16])
def test_append_position_past_the_cache_is_skipped(tokens):
    nq, nkv, D, max_seq = 4, 2, 128, 32
    rng = np.random.default_rng(0)
    qkv = ops.dev(rng.standard_normal((tokens, (nq + 2 * nkv) * D)).astype(np.float32), torch.float16)
    kc, kbuf, kguard = _guarded((tokens, nkv, max_seq, D), fill=0.0)
    vc, vbuf, vguard = _guarded((tokens, nkv, max_seq, D), fill=0.0)
    q = torch.empty(tokens, nq * D, dtype=torch.float16, device="cuda")
    pos_h = np.arange(tokens, dtype=np.int64)
    pos_h[-1] = max_seq                                   # one token too many
    pos_h[0] = -3 if tokens > 2 else 0                    # and a negative one
    pos = ops.dev(pos_h)
    p = capi.QkvRopeAppendParams(capi.FP16, tokens, nq, 10000.0, ops.kv_layout(nkv, D, max_seq))
    capi.call("qkv_rope_append", p, [qkv.data_ptr(), pos.data_ptr(), 0], [q.data_ptr(), kc.data_ptr(), vc.data_ptr()])
    torch.cuda.synchronize()
    _expect_index_error_then_clear()
    bad = [t for t in range(tokens) if not 0 <= pos_h[t] < max_seq]
    for t in range(tokens):
        row_written = bool((kc[t] != 0).any())
        assert row_written == (t not in bad)
        if t in bad:
            assert not (vc[t] != 0).any()
    assert (kguard == 7).all() and (vguard == 7).all()
    assert torch.isfinite(q).all()                        # q is still produced for every token


def test_linear_qkv_epilogue_skips_out_of_range_append():
    nH, D, H, max_seq = 4, 128, 512, 16
    rng = np.random.default_rng(1)
    x = ops.dev(rng.standard_normal((1, H)).astype(np.float32), torch.float16)
    w = ops.dev(0.05 * rng.standard_normal((3 * nH * D, H)).astype(np.float32), torch.float16)
    kc, _, kguard = _guarded((1, nH, max_seq, D), fill=0.0)
    vc, _, vguard = _guarded((1, nH, max_seq, D), fill=0.0)
    kv = ops.kv_layout(nH, D, max_seq)
    q = ops.linear(x, w, epilogue=3, n_heads=nH, kv=kv, positions=ops.dev(np.array([max_seq], np.int64)), k_cache=kc, v_cache=vc)
    torch.cuda.synchronize()
    _expect_index_error_then_clear()
    assert not (kc != 0).any() and not (vc != 0).any()
    assert (kguard == 7).all() and (vguard == 7).all()
    # the same call with a valid position works and reports nothing
    q2 = ops.linear(x, w, epilogue=3, n_heads=nH, kv=kv, positions=ops.dev(np.array([max_seq - 1], np.int64)), k_cache=kc, v_cache=vc)
    torch.cuda.synchronize()
    assert capi.load().rg_b200_error_state() == 0
    assert (kc[0, :, max_seq - 1] != 0).any()
    assert torch.isfinite(q).all() and torch.isfinite(q2).all()


def test_prefill_gemm_epilogue_checks_positions_and_block_table():
    """The tcgen05 QKV product with the RoPE + append epilogue (more than 64 tokens), paged cache: one token carries a
    position beyond the block table's reach, one sequence's table holds a block id outside the cache."""
    nH, nKV, D, H, page, S, B = 4, 2, 128, 512, 16, 48, 2
    tokens, max_blocks, n_blocks = B * S, 4, 8
    rng = np.random.default_rng(2)
    x = ops.dev(rng.standard_normal((tokens, H)).astype(np.float32), torch.float16)
    w = ops.dev(0.05 * rng.standard_normal(((nH + 2 * nKV) * D, H)).astype(np.float32), torch.float16)
    kc, _, kguard = _guarded((n_blocks, nKV, page, D), fill=0.0)
    vc, _, vguard = _guarded((n_blocks, nKV, page, D), fill=0.0)
    table_h = np.arange(n_blocks, dtype=np.int32).reshape(B, max_blocks)
    table_h[1, 1] = n_blocks + 5                              # sequence 1, tokens 16..31: no such block
    pos_h = np.tile(np.arange(S, dtype=np.int64), B)
    pos_h[5] = page * max_blocks                              # sequence 0, token 5: beyond the table
    kv = ops.kv_layout(nKV, D, 0, page, max_blocks, n_blocks)
    q = ops.linear(x, w, epilogue=3, n_heads=nH, kv=kv, positions=ops.dev(pos_h), table=ops.dev(table_h), k_cache=kc, v_cache=vc,
                   tokens_per_seq=S)
    torch.cuda.synchronize()
    _expect_index_error_then_clear()
    assert (kguard == 7).all() and (vguard == 7).all()
    written = (kc != 0).flatten(1).any(dim=1).cpu().numpy()   # per block
    assert written[[0, 1, 2]].all() and written[4] and written[6]      # blocks of valid tokens
    assert not written[3] and not written[7]                   # S = 48 tokens use three blocks per sequence
    assert not (kc[5] != 0).any()                              # the block the bad table entry displaced stays empty
    assert not (kc[0, :, 5] != 0).any()                        # the token with the bad position wrote nothing
    assert torch.isfinite(q).all()


@pytest.mark.parametrize("nkv", [4, 1])                        # general / grouped-query kernel
def test_decode_attention_clamps_a_length_beyond_the_launch(nkv):
    B, nH, D, max_seq, max_len = 2, 4, 128, 512, 300
    rng = np.random.default_rng(3)
    q = ops.dev(rng.standard_normal((B, nH, D)).astype(np.float32), torch.float16)
    kc = ops.dev(rng.standard_normal((B, nkv, max_seq, D)).astype(np.float32), torch.float16)
    vc = ops.dev(rng.standard_normal((B, nkv, max_seq, D)).astype(np.float32), torch.float16)
    kv = ops.kv_layout(nkv, D, max_seq)
    lens_bad = ops.dev(np.array([100, 100000], np.int64))     # sequence 1 claims far more than max_len
    o, ws = ops.attn_decode(q, kc, vc, lens_bad, kv, max_len)
    torch.cuda.synchronize()
    _expect_index_error_then_clear()
    assert torch.isfinite(o).all()
    want_clamped = onp.attn_decode(q.float().cpu().numpy(), kc.float().cpu().numpy(), vc.float().cpu().numpy(), np.array([100, max_len]))
    np.testing.assert_allclose(o.float().cpu().numpy(), want_clamped, atol=2e-2, rtol=1e-2)
    # the workspace (arrival counters) is ready for the next, valid call
    lens_ok = ops.dev(np.array([100, 299], np.int64))
    o2, _ = ops.attn_decode(q, kc, vc, lens_ok, kv, max_len, ws=ws)
    torch.cuda.synchronize()
    assert capi.load().rg_b200_error_state() == 0
    want = onp.attn_decode(q.float().cpu().numpy(), kc.float().cpu().numpy(), vc.float().cpu().numpy(), np.array([100, 299]))
    np.testing.assert_allclose(o2.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)


def test_decode_attention_rejects_a_block_id_outside_the_cache():
    B, nH, nkv, D, page, max_blocks, n_blocks = 1, 4, 4, 128, 16, 8, 8
    rng = np.random.default_rng(4)
    q = ops.dev(rng.standard_normal((B, nH, D)).astype(np.float32), torch.float16)
    kc = ops.dev(rng.standard_normal((n_blocks, nkv, page, D)).astype(np.float32), torch.float16)
    vc = ops.dev(rng.standard_normal((n_blocks, nkv, page, D)).astype(np.float32), torch.float16)
    table = np.arange(max_blocks, dtype=np.int32).reshape(1, max_blocks)
    table[0, 2] = -1
    table[0, 3] = 1 << 20
    kv = ops.kv_layout(nkv, D, 0, page, max_blocks, n_blocks)
    o, _ = ops.attn_decode(q, kc, vc, ops.dev(np.array([100], np.int64)), kv, 128, table=ops.dev(table))
    torch.cuda.synchronize()
    _expect_index_error_then_clear()
    assert torch.isfinite(o).all()


def test_gather_skips_an_index_outside_the_table():
    table = ops.dev(np.arange(40, dtype=np.float32).reshape(10, 4))
    out = ops.gather(table, ops.dev(np.array([3, 10, -11, -1], np.int64)), 0)
    torch.cuda.synchronize()
    _expect_index_error_then_clear()
    got = out.cpu().numpy()
    np.testing.assert_array_equal(got[0], np.arange(12, 16))
    np.testing.assert_array_equal(got[3], np.arange(36, 40))      # -1 wraps, as in the reference


def test_decode_step_refuses_a_position_past_the_cache_and_a_token_outside_the_vocabulary():
    from refactorgraph_b200.llama import LlamaConfig, decode_step_graph_single_kernel, seeded_weights, weight_inputs
    cfg = LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, max_seq=64, batch=1)
    w16 = seeded_weights(cfg, 0, np.float16)
    g, index = decode_step_graph_single_kernel(cfg)
    ex = g.compiler().compile("cuda", "flat", [])
    for name, _ in weight_inputs(cfg):
        ex.set_input(index[name], w16[name])
    rng = np.random.default_rng(5)
    caches = {}
    for l in range(cfg.layers):
        for nm in ("k_cache", "v_cache"):
            caches[(l, nm)] = rng.standard_normal((1, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16)
            ex.set_input(index[f"l{l}.{nm}"], caches[(l, nm)])
    ex.set_input(index["token"], np.array([7], np.int64))
    ex.set_input(index["pos"], np.array([cfg.max_seq - 1], np.int64))
    ex.run()                                                    # the last position that fits
    assert capi.load().rg_b200_error_state() == 0
    first = ex.get_output(index["next"]).copy()
    ex.run()                                                    # the step advanced pos to max_seq: this one must do nothing
    _expect_index_error_then_clear()
    np.testing.assert_array_equal(ex.get_output(index["next"]), first)
    ex.set_input(index["pos"], np.array([10], np.int64))
    ex.set_input(index["token"], np.array([cfg.vocab], np.int64))
    ex.run()
    _expect_index_error_then_clear()
    ex.set_input(index["token"], np.array([7], np.int64))      # and the workspace still works
    ex.run()
    assert capi.load().rg_b200_error_state() == 0
    assert 0 <= int(ex.get_output(index["next"]).ravel()[0]) < cfg.vocab
