"""Pins the compact KV cache (q8 K + TurboQuant-3 V) on the reference's OWN CUDA kernels.

The reference states this arithmetic in CUDA only (src/kernels/cuda/cuda_engine.cu:199-299,
8224-8314, 8382-8454) and keeps no vectors for it.  oracle/_ref/librl_refcuda.so is that
translation unit compiled where it lies, with the reference's flags (fast math included), behind a
shim that launches store_k_q8_th_k, store_v_tq3_th_k, the two dequantise kernels and
qk_attn_decode_tq_gqa_k.  Compared here on the same seeded rows:
  * the library's codes and scales (layout of two 128-point blocks without signs, the reference's),
  * the C restatement's codes and scales,
  * the dequantised fp16 window, and the decode output.
The reference divides with fast-math approximations (x / s, 1 / rms), the library and the
restatement with IEEE division, so a code that sits on a rounding boundary may differ by one step:
the bound is >= 99.9 % equal codes and no difference larger than one level.
"""
import numpy as np
import pytest
import torch

from helpers import ATTN_MAX_ABS, ATTN_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

N_Q, N_KV, HD = 24, 4, 256
MIN_EQUAL = 0.999


@pytest.fixture(scope="module")
def refcuda():
    from oracle import ReferenceCuda
    if not ReferenceCuda.available():
        pytest.skip("oracle/_ref/librl_refcuda.so not built (reference tree or nvcc absent at build time)")
    return ReferenceCuda()


def _rows(seed, n):
    gen = torch.Generator().manual_seed(seed)
    k = torch.randn(n, N_KV, HD, generator=gen)
    v = torch.randn(n, N_KV, HD, generator=gen)
    k[3] *= 1e-3                                   # a small row, an outlier, a large row
    k[7, 1, 11] = 40.0
    v[9] *= 30.0
    return k, v, gen


def _unpack3(codes):
    """u8 [..., 96] (8 indices LSB-first per 3 bytes) -> indices [..., 256]."""
    c = codes.astype(np.uint32).reshape(*codes.shape[:-1], 32, 3)
    w = c[..., 0] | (c[..., 1] << 8) | (c[..., 2] << 16)
    return np.stack([(w >> (3 * j)) & 7 for j in range(8)], axis=-1).reshape(*codes.shape[:-1], 256).astype(np.int32)


def _f16(bits):
    return np.ascontiguousarray(bits).view(np.float16).astype(np.float32)


def _close_codes(name, ours, ref, max_step=1):
    ours = ours.astype(np.int32)
    ref = ref.astype(np.int32)
    eq = float((ours == ref).mean())
    step = int(np.abs(ours - ref).max())
    print("%s: %.5f %% equal, largest difference %d" % (name, 100 * eq, step))
    assert eq >= MIN_EQUAL, (name, eq)
    assert step <= max_step, (name, step)


def _close_scales(name, ours_bits, ref_bits):
    a, b = _f16(ours_bits), _f16(ref_bits)
    eq = float((np.ascontiguousarray(ours_bits).view(np.uint16) == np.ascontiguousarray(ref_bits).view(np.uint16)).mean())
    rel = float(np.abs(a - b).max() / np.abs(b).max())
    print("%s: %.5f %% equal, max relative difference %.2e" % (name, 100 * eq, rel))
    assert eq >= MIN_EQUAL, (name, eq)
    # never more than one fp16 step apart
    assert np.all(np.abs(a - b) <= np.abs(b) * 2.0 ** -10), name


def test_store_codes_match_the_reference_kernels(refcuda, oracle):
    from rapidllm_b200 import _lib, ops
    n = 4096
    k, v, gen = _rows(31, n)
    rk_q, rk_sc, rv_codes, rv_sc = refcuda.compact_store(k.numpy(), v.numpy())
    # the library
    n_pages = n // 64
    table = torch.randperm(n_pages, generator=gen).int().cuda()
    pool = ops.new_compact_pool(n_pages, N_KV)
    ops.kv_compact_append(pool, table, k.cuda(), v.cuda(), 128, None, pos0=0)
    _lib.check_device()
    k_q, k_sc, v_codes, v_sc = (x.cpu().numpy() for x in ops.kv_compact_gather(pool, table, n, 128))
    _close_codes("library K codes", k_q, rk_q)
    _close_scales("library K scales", k_sc.view(np.uint16), rk_sc)
    _close_codes("library V codes", _unpack3(v_codes), _unpack3(rv_codes))
    _close_scales("library V scales", v_sc.view(np.uint16), rv_sc)
    # the C restatement the other compact-KV tests compare with
    ok_q, ok_sc, ov_codes, ov_sc = oracle.compact_store(k.numpy(), v.numpy(), 128, None)
    _close_codes("restatement K codes", ok_q, rk_q)
    _close_scales("restatement K scales", ok_sc, rk_sc)
    _close_codes("restatement V codes", _unpack3(ov_codes), _unpack3(rv_codes))
    _close_scales("restatement V scales", ov_sc, rv_sc)


def test_dequantised_window_matches_the_reference_kernels(refcuda, oracle):
    """Same codes in, fp16 window out: reference kernels vs the restatement vs rl_kv_compact_to_f16."""
    from rapidllm_b200 import _lib, ops
    n = 640
    k, v, gen = _rows(32, n)
    codes = refcuda.compact_store(k.numpy(), v.numpy())
    rk16, rv16 = refcuda.compact_dequant(*codes)
    ok, ov = oracle.compact_dequant(*codes, 128, None)
    ok16, ov16 = ok.astype(np.float16), ov.astype(np.float16)
    # K = scale * int8 exactly in fp32, then one rounding: identical
    assert np.array_equal(rk16.view(np.uint16), ok16.view(np.uint16))
    # V goes through 7 butterfly stages; the reference's tree and ours add in different orders
    dv = np.abs(rv16.astype(np.float32) - ov16.astype(np.float32))
    print("dequantised V: max-abs %.3e (fp16 step at |v| ~ 4 is 3.9e-3)" % dv.max())
    assert dv.max() <= 2.0 ** -7 * max(1.0, float(np.abs(ov).max()) / 4)
    # the library's window rebuild over its own store of the same rows
    n_pages = n // 64
    table = torch.randperm(n_pages, generator=gen).int().cuda()
    pool = ops.new_compact_pool(n_pages, N_KV)
    ops.kv_compact_append(pool, table, k.cuda(), v.cuda(), 128, None, pos0=0)
    kp, vp = ops.new_pool(n_pages, N_KV), ops.new_pool(n_pages, N_KV)
    dtable = torch.randperm(n_pages, generator=gen).int().cuda()
    ops.kv_compact_to_f16(pool, table, kp, vp, dtable, n, 0, 0, 128, None)
    _lib.check_device()
    lk = ops.kv_gather(kp, dtable, n).cpu().numpy().astype(np.float32)
    lv = ops.kv_gather(vp, dtable, n).cpu().numpy().astype(np.float32)
    rk, rv = rk16.astype(np.float32), rv16.astype(np.float32)
    # the library stored with IEEE division: its codes differ from the reference's on < 0.1 % of
    # the entries, by one level; compare the windows in relative L2 and on the bulk of entries
    print("window K rel-l2 %.3e, V rel-l2 %.3e" % (rel_l2(lk, rk), rel_l2(lv, rv)))
    assert rel_l2(lk, rk) <= 2e-3 and rel_l2(lv, rv) <= 2e-2
    assert float((np.abs(lk - rk) <= 2.0 ** -9 * np.maximum(1.0, np.abs(rk))).mean()) >= MIN_EQUAL


@pytest.mark.parametrize("n", [1, 33, 700, 4096])
def test_decode_matches_the_reference_kernel(refcuda, n):
    """qk_attn_decode_tq_gqa_k over the reference's store vs rl_attn_decode over the library's store."""
    from rapidllm_b200 import _lib, ops
    k, v, gen = _rows(33 + n, max(n, 16))
    k, v = k[:n], v[:n]
    q = torch.randn(N_Q, HD, generator=gen)
    ref = refcuda.attn_decode_tq(q.numpy(), *refcuda.compact_store(k.numpy(), v.numpy()))
    n_pages = (n + 63) // 64 + 1
    table = torch.randperm(n_pages, generator=gen).int()[: (n + 63) // 64].cuda()
    pool = ops.new_compact_pool(n_pages, N_KV)
    pool.fill_(0xFF)
    ops.kv_compact_append(pool, table, k.cuda(), v.cuda(), 128, None, pos0=0)
    sl = torch.tensor([n], dtype=torch.int32, device="cuda")
    o = ops.attn_decode(q.cuda().unsqueeze(0), pool, None, table.unsqueeze(0), sl, None, wht_len=128, signs=None)
    _lib.check_device()
    o = o[0].cpu().numpy()
    print("decode over %d tokens vs the reference kernel: max-abs %.3e rel-l2 %.3e" %
          (n, np.abs(o - ref).max(), rel_l2(o, ref)))
    assert np.isfinite(o).all()
    assert np.abs(o - ref).max() <= ATTN_MAX_ABS
    assert rel_l2(o, ref) <= ATTN_REL_L2
