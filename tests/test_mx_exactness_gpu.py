"""Dequantisation checked on the product decode kernel itself (through the C ABI), not on a side
kernel: with a context of one token the softmax weight is exactly 1, so the attention output IS the
dequantised V row and the log-sum-exp IS one dequantised K element times the softmax scale.

Spec the kernel is held to: ``oracle/paged_decode_oracle.py`` (E4M3 / E2M1 code tables, E8M0 =
2**(e - 127) for every finite byte).  The reference project defines none of the microscaling
formats; its E4M3 recipe is ``tests/test_kernels_misc.py:51-59`` there."""
import numpy as np
import pytest
import torch

from helpers import to_oracle
from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu

PAGE = 16


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


def _single_token_workload(v_fmt, d, hkv, n_seq, e_lo, e_hi, spread, seed, q_dtype, group=2, one_hot=False,
                           k_exp=(-2, 2)):
    """``n_seq`` sequences of ONE token each.  V codes walk through every code of the format, V block
    exponents walk through [e_lo, e_hi] per (sequence, head) with the blocks of one token at most
    ``spread`` apart; every other slot of every page is poisoned (NaN codes, NaN scale bytes)."""
    from cuda_b200 import workloads as W
    g = torch.Generator().manual_seed(seed)
    nb = d // 32
    perm = torch.randperm(n_seq, generator=g)
    kc = torch.full((n_seq, hkv, d, PAGE), W.POISON_E4M3, dtype=torch.uint8)
    dv = d if v_fmt == "fp8_e4m3" else d // 2
    vc = torch.full((n_seq, hkv, dv, PAGE), W.POISON_E4M3, dtype=torch.uint8)
    ks = torch.full((n_seq, hkv, nb, PAGE), W.POISON_E8M0, dtype=torch.uint8)
    vs = torch.full((n_seq, hkv, nb, PAGE), W.POISON_E8M0, dtype=torch.uint8)
    # K: random finite codes, block exponents in k_exp
    kcodes = torch.randint(0, 256, (n_seq, hkv, d), generator=g).to(torch.uint8)
    kcodes[(kcodes & 0x7F) == 0x7F] = 0x38
    kc[perm, :, :, 0] = kcodes
    ks[perm, :, :, 0] = torch.randint(k_exp[0] + 127, k_exp[1] + 128, (n_seq, hkv, nb), generator=g).to(torch.uint8)
    # V: every code in turn
    idx = torch.arange(n_seq * hkv * d).view(n_seq, hkv, d)
    if v_fmt == "fp8_e4m3":
        vcodes = ((idx * 37 + idx // 256) % 256).to(torch.uint8)
        vcodes[(vcodes & 0x7F) == 0x7F] = 0x08
        vc[perm, :, :, 0] = vcodes
    else:
        nib = ((idx * 5 + idx // 16) % 16).to(torch.uint8).view(n_seq, hkv, d // 2, 2)
        vc[perm, :, :, 0] = nib[..., 0] | (nib[..., 1] << 4)
    span = e_hi - e_lo + 1
    base = (torch.arange(n_seq * hkv).view(n_seq, hkv, 1) * 7) % span + e_lo            # per (sequence, head)
    off = -torch.randint(0, spread + 1, (n_seq, hkv, nb), generator=g)
    off[:, :, 0] = 0
    e = (base + off).clamp(e_lo, e_hi)
    vs[perm, :, :, 0] = (e + 127).to(torch.uint8)
    hq = hkv * group
    if one_hot:
        q = torch.zeros(n_seq, hq, d)
        q[torch.arange(n_seq), :, torch.arange(n_seq) % d] = 1.0
    else:
        q = torch.randn(n_seq, hq, d, generator=g)
    return W.DecodeWorkload(
        name="mx_single_token", query=q.to(q_dtype), key_cache=kc, value_cache=vc, k_scale=ks, v_scale=vs,
        block_tables=perm.view(n_seq, 1).to(torch.int32), context_lens=torch.ones(n_seq, dtype=torch.int32),
        cu_q_lens=None, page_size=PAGE, head_dim=d, num_q_heads=hq, num_kv_heads=hkv, k_format="fp8_e4m3",
        v_format=v_fmt, k_scale_mode="mx_e8m0", v_scale_mode="mx_e8m0", softmax_scale=1.0, max_q_len=1)


@pytest.mark.parametrize("q_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("v_fmt,d,e_lo,e_hi", [("fp8_e4m3", 128, -30, 20), ("fp8_e4m3", 64, -30, 20),
                                               ("fp4_e2m1", 128, -30, 20), ("fp8_e4m3", 128, -90, 90),
                                               ("fp4_e2m1", 64, -90, 90)])
def test_v_dequant_bit_exact_on_decode_kernel(ops, v_fmt, d, e_lo, e_hi, q_dtype):
    """Context length 1: out == dequantised V, bit for bit, for every element code and every block
    exponent of the range (blocks of one token up to 2^14 apart)."""
    wl = _single_token_workload(v_fmt, d, hkv=8, n_seq=64, e_lo=e_lo, e_hi=e_hi, spread=14, seed=3, q_dtype=q_dtype)
    kv = to_oracle(wl)
    out = ops.run_workload(wl.to("cuda"), check_status=True).cpu()
    group = wl.num_q_heads // wl.num_kv_heads
    for s in range(wl.num_seqs):
        _, v = O.gather_sequence(kv, s)                       # [Hkv, 1, D] fp32
        want = v[:, 0].repeat_interleave(group, dim=0).to(q_dtype)
        assert torch.equal(out[s], want), (s, (out[s].float() - want.float()).abs().max())
    # every code of the format and every exponent of the range took part
    codes = wl.value_cache[:, :, :, 0]
    assert len(torch.unique(codes & 0x0F if v_fmt == "fp4_e2m1" else codes)) >= (16 if v_fmt == "fp4_e2m1" else 254)
    assert len(torch.unique(wl.v_scale[:, :, :, 0])) >= min(e_hi - e_lo + 1, 64 * 8) - 14


def _ulp(x):
    return np.spacing(np.abs(x.numpy()).astype(np.float32))


@pytest.mark.parametrize("d", [64, 128])
def test_k_dequant_through_lse_on_decode_kernel(ops, d):
    """One-hot fp32 queries, context length 1, softmax scale 1: the returned log-sum-exp is the
    dequantised K element (E4M3 code times 2^(e-127) of its block), to a few ulp (the kernel works in
    base 2 and converts back)."""
    wl = _single_token_workload("fp8_e4m3", d, hkv=4, n_seq=2 * d, e_lo=0, e_hi=0, spread=0, seed=5,
                                q_dtype=torch.float32, one_hot=True, k_exp=(-24, 16))
    kv = to_oracle(wl)
    _, lse = ops.run_workload(wl.to("cuda"), return_lse=True, check_status=True)
    lse = lse.cpu()
    group = wl.num_q_heads // wl.num_kv_heads
    for s in range(wl.num_seqs):
        k, _ = O.gather_sequence(kv, s)                       # [Hkv, 1, D]
        want = k[:, 0, s % d].repeat_interleave(group)
        err = (lse[s] - want).abs().numpy()
        assert (err <= 4 * _ulp(want)).all(), (s, lse[s], want)


@pytest.mark.parametrize("v_fmt", ["fp8_e4m3", "fp4_e2m1"])
@pytest.mark.parametrize("spread", [6, 50])
def test_mx_wide_exponent_range_parity(ops, v_fmt, spread):
    """MX caches whose V block exponents cover [-30, +20] (small and large V alike) against the
    oracle.  Outputs are as large as 2^20 here, so the stated bf16 tolerance is taken relative to the
    largest output of each row.  spread 50: the blocks of one token differ by up to 2^50, a block more
    than 2^14 below its token's largest contributes zero, which is far inside the tolerance."""
    from cuda_b200 import workloads as W
    lens = [1, 17, 300, 64, 1000, 33]
    wl = W.build_workload("mxwide", context_lens=lens, q_lens=None, num_q_heads=16, num_kv_heads=4, head_dim=128,
                          page_size=16, q_dtype=torch.bfloat16, v_format=v_fmt, scale_mode="mx_e8m0",
                          pool_factor=1.3, seed=13)
    g = torch.Generator().manual_seed(14)
    pool = wl.v_scale.shape[0]
    base = torch.randint(-30 + spread if spread < 50 else 20, 21, (pool, 4, 1, 16), generator=g)
    e = base - torch.randint(0, spread + 1, (pool, 4, 4, 16), generator=g)
    live = wl.v_scale != W.POISON_E8M0
    wl.v_scale = torch.where(live, (e.clamp(-30, 20) + 127).to(torch.uint8), wl.v_scale)
    kv = to_oracle(wl)
    ref = O.ref_paged_decode(wl.query, kv, wl.softmax_scale)
    out = ops.run_workload(wl.to("cuda"), check_status=True).float().cpu()
    assert torch.isfinite(out).all()
    scale = ref.abs().amax(dim=-1, keepdim=True).clamp_min(1.0)
    err = (out - ref).abs() / scale
    assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())


def test_scale_byte_outside_supported_range_sets_status(ops):
    """E8M0 V bytes below 32 or above 223 (2^-95 .. 2^96) are reported, not silently mangled."""
    wl = _single_token_workload("fp8_e4m3", 128, hkv=8, n_seq=8, e_lo=-4, e_hi=4, spread=2, seed=9,
                                q_dtype=torch.bfloat16)
    wl.v_scale[int(wl.block_tables[3, 0]), 2, :, 0] = 10
    g = wl.to("cuda")
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(wl.num_seqs, wl.num_q_heads, wl.num_kv_heads,
                                                              wl.head_dim, wl.page_size, 1, 0)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    ops.run_workload(g, workspace=ws)
    assert ops.decode_status(ws) & ops.L.ST_SCALE_RANGE
    wl.v_scale[int(wl.block_tables[3, 0]), 2, :, 0] = 127
    ops.run_workload(wl.to("cuda"), workspace=ws)
    assert ops.decode_status(ws) == 0
