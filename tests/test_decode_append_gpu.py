"""Decode-step glue (RoPE + quantise of the new token, append to the FP8 KV cache) against its restatement: the codes
are bit-exact, every cache byte outside the appended rows is untouched, and a generation loop of append + fa_decode
steps stays within the attention tolerance of the fp64 restatement over the cache the restatement built itself."""
import math

import numpy as np
import pytest
import torch

import oracle as O
from oracle import glue

pytestmark = pytest.mark.gpu


def rope_tables(rows, hd, theta=10000.0):
    from goml_b200 import block_glue as BG
    cos = torch.empty(rows, hd // 2, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    BG.RopeTable(cos.data_ptr(), sin.data_ptr(), rows, hd, theta)
    torch.cuda.synchronize()
    return cos, sin


def make_inputs(name, B, Hq, Hkv, Smax, hd):
    qkv = O.round_bf16(O.seeded_normal("qkv", (B, (Hq + 2 * Hkv) * hd), config=name)).astype(np.float32)
    k, sk, _ = O.quantize_f32(O.seeded_normal("k", (B, Hkv, Smax, hd), config=name))
    v, sv, _ = O.quantize_f32(O.seeded_normal("v", (B, Hkv, Smax, hd), config=name))
    return qkv, k, v, float(sk), float(sv)


def run_append(qkv, cos, sin, positions, k, v, sk, sv, Hq, Hkv, hd, table=None, page=0):
    from goml_b200 import block_glue as BG
    B = qkv.shape[0]
    qkv_d = torch.from_numpy(qkv).cuda().bfloat16()
    pos_d = torch.from_numpy(np.asarray(positions, np.int32)).cuda()
    kd, vd = torch.from_numpy(k.copy()).cuda(), torch.from_numpy(v.copy()).cuda()
    q = torch.full((B, Hq, hd), 0xAA, dtype=torch.uint8, device="cuda")
    sc = torch.tensor([7.0, 7.0, sk, sv], dtype=torch.float32, device="cuda")
    lens = torch.full((B,), -7, dtype=torch.int32, device="cuda")
    kw = {}
    if table is not None:
        td = torch.from_numpy(np.ascontiguousarray(table, np.int32)).cuda()
        kw = dict(block_table=td.data_ptr(), page_size=page, max_pages_per_seq=table.shape[1], num_pages=k.shape[0])
    BG.DecodeRopeAppend(qkv_d.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos_d.data_ptr(), q.data_ptr(), sc.data_ptr(),
                        sc.data_ptr() + 4, kd.data_ptr(), vd.data_ptr(), sc.data_ptr() + 8, sc.data_ptr() + 12, B, Hq, Hkv, hd,
                        0 if table is not None else k.shape[2], cos.shape[0], seq_lens_out=lens.data_ptr(), **kw)
    torch.cuda.synchronize()
    return q.cpu().numpy(), float(sc[0].item()), float(sc[1].item()), kd.cpu().numpy(), vd.cpu().numpy(), lens.cpu().numpy()


@pytest.mark.parametrize("B,Hq,Hkv,Smax,hd", [(5, 8, 2, 96, 128), (3, 4, 4, 64, 64), (64, 32, 8, 256, 128)])
def test_codes_and_cache_rows_bit_exact(cuda, built_libs, B, Hq, Hkv, Smax, hd):
    name = f"append{B}_{Hq}_{Hkv}_{Smax}_{hd}"
    qkv, k, v, sk, sv = make_inputs(name, B, Hq, Hkv, Smax, hd)
    cos, sin = rope_tables(Smax, hd)
    rng = np.random.default_rng(B + Smax)
    positions = rng.integers(0, Smax, size=B)
    positions[0] = Smax - 1
    if B > 2:
        positions[1] = -1            # an inactive slot
        positions[2] = Smax          # a full cache
    got = run_append(qkv, cos, sin, positions, k, v, sk, sv, Hq, Hkv, hd)
    ref = glue.decode_rope_append(qkv, cos.cpu().numpy(), sin.cpu().numpy(), positions, k, v, sk, sv, Hq, Hkv, hd)
    assert np.array_equal(got[0], ref[0])
    assert got[1] == float(ref[1]) and got[2] == float(ref[2])
    assert np.array_equal(got[3], ref[3]) and np.array_equal(got[4], ref[4])     # whole caches: appended rows and all the rest
    assert np.array_equal(got[5], ref[5])


def test_values_beyond_the_cache_scale_saturate(cuda, built_libs):
    B, Hq, Hkv, Smax, hd = 2, 4, 2, 64, 64
    qkv, k, v, sk, sv = make_inputs("append-sat", B, Hq, Hkv, Smax, hd)
    cos, sin = rope_tables(Smax, hd)
    sk, sv = 1e-9, 1e-9                                      # every new value is far beyond 448 * scale
    got = run_append(qkv, cos, sin, [3, 9], k, v, sk, sv, Hq, Hkv, hd)
    ref = glue.decode_rope_append(qkv, cos.cpu().numpy(), sin.cpu().numpy(), [3, 9], k, v, sk, sv, Hq, Hkv, hd)
    assert np.array_equal(got[3], ref[3]) and np.array_equal(got[4], ref[4])
    assert set(np.unique(got[4][0, :, 3] & 0x7F)) <= {0x7E, 0x00}           # +-448 (or an exact zero), never NaN


def test_paged_append_writes_the_same_rows(cuda, built_libs):
    from tests.test_fa_decode_gpu import to_pages
    B, Hq, Hkv, Smax, hd, page = 4, 8, 2, 256, 128, 64
    qkv, k, v, sk, sv = make_inputs("append-paged", B, Hq, Hkv, Smax, hd)
    cos, sin = rope_tables(Smax, hd)
    rng = np.random.default_rng(11)
    kp, table = to_pages(k, page, rng)
    vp = np.full_like(kp, 0xFF)
    for b in range(B):
        for j in range(Smax // page):
            vp[table[b, j]] = v[b, :, j * page:(j + 1) * page]
    positions = np.array([0, 63, 64, 255], np.int32)
    table_dev = table.copy()
    table_dev[2, 1] = 10 ** 6                               # no page behind position 64 of sequence 2: nothing written
    got = run_append(qkv, cos, sin, positions, kp, vp, sk, sv, Hq, Hkv, hd, table=table_dev, page=page)
    ref = glue.decode_rope_append(qkv, cos.cpu().numpy(), sin.cpu().numpy(), positions, k, v, sk, sv, Hq, Hkv, hd)
    assert np.array_equal(got[0], ref[0]) and np.array_equal(got[5], ref[5])
    want_k, want_v = kp.copy(), vp.copy()
    for b in (0, 1, 3):
        pos = int(positions[b])
        want_k[table[b, pos // page], :, pos % page] = ref[3][b, :, pos]
        want_v[table[b, pos // page], :, pos % page] = ref[4][b, :, pos]
    assert np.array_equal(got[3], want_k) and np.array_equal(got[4], want_v)


def test_generation_loop_append_then_decode(cuda, built_libs, fa_ctx):
    # four steps of: project (random rows here) -> append -> attend; the device cache must equal the restatement's cache
    # after every step and the attention output must stay within the attention tolerance
    from goml_b200 import block_glue as BG
    B, Hq, Hkv, Smax, hd = 3, 8, 2, 128, 128
    _, k, v, sk, sv = make_inputs("append-loop", B, Hq, Hkv, Smax, hd)
    cos, sin = rope_tables(Smax, hd)
    cos_h, sin_h = cos.cpu().numpy(), sin.cpu().numpy()
    positions = np.array([5, 64, 123], np.int32)
    kd, vd = torch.from_numpy(k.copy()).cuda(), torch.from_numpy(v.copy()).cuda()
    sc = torch.tensor([0.0, 0.0, sk, sv], dtype=torch.float32, device="cuda")
    q = torch.empty((B, Hq, hd), dtype=torch.uint8, device="cuda")
    lens = torch.zeros((B,), dtype=torch.int32, device="cuda")
    o = torch.empty((B, Hq, hd), dtype=torch.float16, device="cuda")
    lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
    kr, vr = k, v
    for step in range(4):
        qkv = O.round_bf16(O.seeded_normal(f"qkv{step}", (B, (Hq + 2 * Hkv) * hd), config="append-loop")).astype(np.float32)
        qkv_d = torch.from_numpy(qkv).cuda().bfloat16()
        pos_d = torch.from_numpy(positions).cuda()
        BG.DecodeRopeAppend(qkv_d.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos_d.data_ptr(), q.data_ptr(), sc.data_ptr(),
                            sc.data_ptr() + 4, kd.data_ptr(), vd.data_ptr(), sc.data_ptr() + 8, sc.data_ptr() + 12, B, Hq, Hkv, hd,
                            Smax, Smax, seq_lens_out=lens.data_ptr())
        fa_ctx.Decode(q.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(), lens.data_ptr(), B, Hq, Hkv, hd, Smax, 0,
                      1.0 / math.sqrt(hd), 1.0, scale_q_dev=sc.data_ptr(), scale_k_dev=sc.data_ptr() + 8, scale_v_dev=sc.data_ptr() + 12)
        torch.cuda.synchronize()
        fa_ctx.DeviceStatus()
        qc, qs, _, kr, vr, sl = glue.decode_rope_append(qkv, cos_h, sin_h, positions, kr, vr, sk, sv, Hq, Hkv, hd)
        assert np.array_equal(kd.cpu().numpy(), kr) and np.array_equal(vd.cpu().numpy(), vr) and np.array_equal(q.cpu().numpy(), qc)
        ref, rl = glue.decode_attention_f64(qc, kr, vr, sl, float(qs) * sk / math.sqrt(hd), sv)
        maxabs, meanrel = O.error_stats(o.double().cpu().numpy(), ref)
        assert maxabs <= 2e-2 and meanrel <= 1e-2 and np.abs(lse.double().cpu().numpy() - rl).max() <= 5e-3, (step, maxabs, meanrel)
        positions = positions + 1
