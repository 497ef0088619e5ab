"""Decode step (one new token per sequence, FP8 KV cache, grouped-query heads) against the fp64 restatement.

Tolerance: the stated bar of the path (max-abs <= 2e-2, mean relative <= 1e-2 on the fp16 output; LSE within 5e-3).
The reference has no implementation of this step (design notes only), so there is no golden vector to pin:
parity unpinned; the restatement is the single-row case of the attention restatement the prefill tests use, and
one test below checks the decode kernel against the prefill kernel's last row on the same cache.
"""
import math

import numpy as np
import pytest
import torch

import oracle as O
from oracle import glue

pytestmark = pytest.mark.gpu


def run_decode(ctx, q, kc, vc, seq_lens, scale, v_descale=1.0, s_max=None, uniform_len=None):
    B, Hq, D = q.shape
    Hkv, Smax = kc.shape[1], kc.shape[2]
    qd, kd, vd = (torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (q, kc, vc))
    o = torch.full((B, Hq, D), float("nan"), dtype=torch.float16, device="cuda")
    lse = torch.full((B, Hq), float("nan"), dtype=torch.float32, device="cuda")
    sl = None if uniform_len is not None else torch.from_numpy(np.asarray(seq_lens, np.int32)).cuda()
    ctx.Decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), 0 if sl is None else sl.data_ptr(),
               B, Hq, Hkv, D, Smax, uniform_len or 0, scale, v_descale)
    torch.cuda.synchronize()
    ctx.DeviceStatus()
    return o.double().cpu().numpy(), lse.double().cpu().numpy()


def make_case(name, B, Hq, Hkv, Smax, D):
    qf = O.seeded_normal("q", (B, Hq, D), config=name)
    kf = O.seeded_normal("k", (B, Hkv, Smax, D), config=name)
    vf = O.seeded_normal("v", (B, Hkv, Smax, D), config=name)
    (q, sq, _), (k, sk, _), (v, sv, _) = (O.quantize_f32(t) for t in (qf, kf, vf))
    return q, k, v, float(sq), float(sk), float(sv)


@pytest.mark.parametrize("B,Hq,Hkv,Smax,D", [(2, 8, 2, 300, 128), (3, 4, 4, 64, 64), (1, 16, 1, 1000, 128), (5, 12, 4, 129, 64),
                                             (2, 32, 8, 2048, 128)])
def test_decode_matches_restatement(cuda, built_libs, fa_ctx, B, Hq, Hkv, Smax, D):
    name = f"decode{B}_{Hq}_{Hkv}_{Smax}_{D}"
    q, k, v, sq, sk, sv = make_case(name, B, Hq, Hkv, Smax, D)
    rng = np.random.default_rng(B * 131 + Smax)
    seq_lens = rng.integers(1, Smax + 1, size=B)
    seq_lens[0] = Smax                       # one full-length sequence
    scale = sq * sk / math.sqrt(D)
    got, lse = run_decode(fa_ctx, q, k, v, seq_lens, scale, sv)
    ref, rl = glue.decode_attention_f64(q, k, v, seq_lens, scale, sv)
    assert np.isfinite(got).all()
    maxabs, meanrel = O.error_stats(got, ref)
    assert maxabs <= 2e-2 and meanrel <= 1e-2, (maxabs, meanrel)
    assert np.abs(lse - rl).max() <= 5e-3


def test_uniform_length_and_empty_sequences(cuda, built_libs, fa_ctx):
    B, Hq, Hkv, Smax, D = 3, 8, 2, 200, 128
    q, k, v, sq, sk, sv = make_case("decode-uniform", B, Hq, Hkv, Smax, D)
    scale = sq * sk / math.sqrt(D)
    got, lse = run_decode(fa_ctx, q, k, v, None, scale, sv, uniform_len=77)
    ref, rl = glue.decode_attention_f64(q, k, v, [77] * B, scale, sv)
    maxabs, meanrel = O.error_stats(got, ref)
    assert maxabs <= 2e-2 and meanrel <= 1e-2 and np.abs(lse - rl).max() <= 5e-3
    # a sequence with no visible key: O = 0, LSE = -inf; lengths beyond s_max are clamped
    got, lse = run_decode(fa_ctx, q, k, v, [0, 50, 10 ** 6], scale, sv)
    ref, rl = glue.decode_attention_f64(q, k, v, [0, 50, Smax], scale, sv)
    assert np.all(got[0] == 0) and np.all(np.isneginf(lse[0]))
    maxabs, meanrel = O.error_stats(got[1:], ref[1:])
    assert maxabs <= 2e-2 and meanrel <= 1e-2 and np.abs(lse[1:] - rl[1:]).max() <= 5e-3


def test_decode_equals_last_row_of_prefill(cuda, built_libs, fa_ctx):
    # the same cache through the prefill kernel (causal): its last query row is the decode step's answer
    from tests.gpu_util import run_attention
    BH, S, D = 4, 320, 128
    q, k, v, sq, sk, sv = make_case("decode-vs-prefill", BH, 1, 1, S, D)      # q: [BH, 1, D] (one query head per kv head)
    qfull = np.zeros((BH, S, D), np.uint8)
    qfull[:, S - 1] = q[:, 0]
    scale = sq * sk / math.sqrt(D)
    o_pre, lse_pre = run_attention(fa_ctx, qfull, k[:, 0], v[:, 0], causal=1, scale=scale, v_descale=sv, entry="ex")
    got, lse = run_decode(fa_ctx, q, k, v, [S] * BH, scale, sv)
    assert np.abs(got[:, 0] - o_pre[:, S - 1]).max() <= 2e-3
    assert np.abs(lse[:, 0] - lse_pre[:, S - 1]).max() <= 1e-4


def test_rejects_bad_arguments(cuda, built_libs, fa_ctx):
    from goml_b200 import fa_forward as F
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    for args, code in [((p, p, p, p, 0, 0, 1, 6, 4, 128, 64, 64, 1.0), F.FA_ERR_UNSUPPORTED_SHAPE),    # 6 % 4 != 0
                       ((p, p, p, p, 0, 0, 1, 32, 1, 128, 64, 64, 1.0), F.FA_ERR_UNSUPPORTED_SHAPE),   # 32 query heads per kv head
                       ((p, p, p, p, 0, 0, 1, 8, 2, 96, 64, 64, 1.0), F.FA_ERR_UNSUPPORTED_HD),
                       ((p, p, p, p, 0, 0, 1, 8, 2, 128, 64, 65, 1.0), F.FA_ERR_INVALID_ARG),          # seq_len > s_max
                       ((p, 0, p, p, 0, 0, 1, 8, 2, 128, 64, 64, 1.0), F.FA_ERR_INVALID_ARG)]:
        with pytest.raises(F.FAError) as e:
            fa_ctx.Decode(*args)
        assert e.value.status == code, (args, e.value.status)


def to_pages(cache, page, rng, spare=3):
    """Contiguous [B, Hkv, S, D] cache -> (pool [P, Hkv, page, D], table [B, S/page]) with the pages of every
    sequence scattered over a pool that also holds `spare` unused pages full of NaN codes."""
    B, Hkv, S, D = cache.shape
    per_seq = S // page
    P = B * per_seq + spare
    pool = np.full((P, Hkv, page, D), 0x7F, np.uint8)
    table = rng.permutation(P)[:B * per_seq].astype(np.int32).reshape(B, per_seq)
    for b in range(B):
        for j in range(per_seq):
            pool[table[b, j]] = cache[b, :, j * page:(j + 1) * page]
    return pool, table


@pytest.mark.parametrize("B,Hq,Hkv,S,D,page", [(3, 8, 2, 512, 128, 64), (2, 16, 4, 1024, 64, 256), (4, 8, 8, 384, 128, 128),
                                               (2, 32, 8, 4096, 128, 512)])
def test_paged_cache_equals_contiguous_cache(cuda, built_libs, fa_ctx, B, Hq, Hkv, S, D, page):
    # the same keys and values behind a block table: same split of the key range, same arithmetic -> identical bits
    name = f"paged{B}_{Hq}_{Hkv}_{S}_{D}_{page}"
    q, k, v, sq, sk, sv = make_case(name, B, Hq, Hkv, S, D)
    rng = np.random.default_rng(S + page)
    seq_lens = rng.integers(1, S + 1, size=B).astype(np.int32)
    seq_lens[0] = S
    scale = sq * sk / math.sqrt(D)
    want, want_lse = run_decode(fa_ctx, q, k, v, seq_lens, scale, sv)
    ref, rl = glue.decode_attention_f64(q, k, v, seq_lens, scale, sv)
    kp, table = to_pages(k, page, rng)
    # one table serves both pools, so V is laid out with K's table
    vp = np.full_like(kp, 0xFF)
    for b in range(B):
        for j in range(S // page):
            vp[table[b, j]] = v[b, :, j * page:(j + 1) * page]
    table_dev = table.copy()
    for b in range(B):                                    # entries past a sequence's pages are never read: poison them
        table_dev[b, (int(seq_lens[b]) + page - 1) // page:] = -12345
    qd, kd, vd, td = (torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (q, kp, vp, table_dev))
    sl = torch.from_numpy(seq_lens).cuda()
    o = torch.full((B, Hq, D), float("nan"), dtype=torch.float16, device="cuda")
    lse = torch.full((B, Hq), float("nan"), dtype=torch.float32, device="cuda")
    fa_ctx.Decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), sl.data_ptr(), B, Hq, Hkv, D, 0, 0,
                  scale, sv, block_table=td.data_ptr(), page_size=page, max_pages_per_seq=S // page, num_pages=kp.shape[0])
    torch.cuda.synchronize()
    fa_ctx.DeviceStatus()
    got, got_lse = o.double().cpu().numpy(), lse.double().cpu().numpy()
    assert np.array_equal(got, want) and np.array_equal(got_lse, want_lse)
    maxabs, meanrel = O.error_stats(got, ref)
    assert maxabs <= 2e-2 and meanrel <= 1e-2 and np.abs(got_lse - rl).max() <= 5e-3


def test_bytes_past_the_sequence_length_are_never_used(cuda, built_libs, fa_ctx):
    # a cache that was allocated and not cleared holds arbitrary bytes past each sequence's end, NaN codes included:
    # the result must be bit-identical to the one over a clean cache
    B, Hq, Hkv, S, D = 4, 8, 2, 300, 128
    q, k, v, sq, sk, sv = make_case("decode-stale", B, Hq, Hkv, S, D)
    seq_lens = np.array([1, 63, 130, 299], np.int32)
    scale = sq * sk / math.sqrt(D)
    want, want_lse = run_decode(fa_ctx, q, k, v, seq_lens, scale, sv)
    k2, v2 = k.copy(), v.copy()
    for b, n in enumerate(seq_lens):
        k2[b, :, n:] = 0x7F
        v2[b, :, n:] = 0xFF
    got, got_lse = run_decode(fa_ctx, q, k2, v2, seq_lens, scale, sv)
    assert np.isfinite(got).all()
    assert np.array_equal(got, want) and np.array_equal(got_lse, want_lse)


def test_paged_rejects_bad_page_size(cuda, built_libs, fa_ctx):
    from goml_b200 import fa_forward as F
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    for kw in (dict(page_size=48, max_pages_per_seq=2, num_pages=4), dict(page_size=64, max_pages_per_seq=0, num_pages=4),
               dict(page_size=64, max_pages_per_seq=2, num_pages=0)):
        with pytest.raises(F.FAError) as e:
            fa_ctx.Decode(p, p, p, p, 0, 0, 1, 8, 2, 128, 0, 64, 1.0, block_table=p, **kw)
        assert e.value.status == F.FA_ERR_INVALID_ARG
