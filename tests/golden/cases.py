"""Input builders shared by ``make_golden.py`` and the tests.

They replay the reference's own test inputs (``tests/test_kernels_misc.py:13-21,26-35,42-64``,
``tests/test_attention.py:76-86``) with the reference's seeding rule
(``tests/conftest.py:31-33``), on the CPU generator so that the same bytes can be rebuilt on
any machine from the seed alone.
"""
import torch

PAGE = 16
DTYPES = {"f16": torch.float16, "bf16": torch.bfloat16}


def paged_cases():
    for dn, dt in DTYPES.items():
        for hd in (64, 128):
            for i, lens in enumerate(([1, 16, 17], [300, 129, 64])):
                yield f"paged_{dn}_d{hd}_l{i}", dt, hd, lens


def fp8_cases():
    for dn, dt in DTYPES.items():
        for hd in (64, 128):
            yield f"fp8_{dn}_d{hd}", dt, hd, [300, 129, 64]


def decode_cases():
    for dn, dt in DTYPES.items():
        for hd in (64, 128):
            for kv_len in (1, 63, 64, 1000):
                yield f"decode_{dn}_d{hd}_s{kv_len}", dt, hd, kv_len


def paged_inputs(dtype, head_dim, context_lens):
    torch.manual_seed(0)
    n, h = len(context_lens), 4
    t = max(context_lens)
    q = torch.randn(n, h, head_dim, dtype=dtype)
    k = torch.randn(n, h, t, head_dim, dtype=dtype)
    v = torch.randn(n, h, t, head_dim, dtype=dtype)
    lens = torch.tensor(context_lens, dtype=torch.int32)
    return q, k, v, lens


def fp8_quantise(k, v):
    h = k.shape[1]
    k_scale = (k.float().abs().amax(dim=(0, 2, 3)) / 448.0).clamp_min(1e-8)
    v_scale = (v.float().abs().amax(dim=(0, 2, 3)) / 448.0).clamp_min(1e-8)
    k8 = (k.float() / k_scale.view(1, h, 1, 1)).to(torch.float8_e4m3fn)
    v8 = (v.float() / v_scale.view(1, h, 1, 1)).to(torch.float8_e4m3fn)
    k_deq = k8.float() * k_scale.view(1, h, 1, 1)
    v_deq = v8.float() * v_scale.view(1, h, 1, 1)
    return k8.view(torch.uint8), v8.view(torch.uint8), k_scale, v_scale, k_deq, v_deq


def decode_inputs(dtype, head_dim, kv_len):
    torch.manual_seed(0)
    q = torch.randn(2, 4, 1, head_dim, dtype=dtype)
    k = torch.randn(2, 4, kv_len, head_dim, dtype=dtype)
    v = torch.randn(2, 4, kv_len, head_dim, dtype=dtype)
    return q, k, v


def rope_cases():
    for dn, dt in DTYPES.items():
        for hd in (64, 128):
            yield f"rope_{dn}_d{hd}", dt, hd, 200


def rope_inputs(dtype, head_dim, seq_len):
    """q, k, v [B, H, S, D] of a causal RoPE attention (``tests/test_attention.py`` of the reference
    builds its RoPE case the same way): the last query row is a decode step over the S cached tokens."""
    torch.manual_seed(0)
    q = torch.randn(2, 4, seq_len, head_dim, dtype=dtype)
    k = torch.randn(2, 4, seq_len, head_dim, dtype=dtype)
    v = torch.randn(2, 4, seq_len, head_dim, dtype=dtype)
    return q, k, v


GQA_ROWS = (0, 37, 99)      # query positions whose reference output rows the fixture keeps


def gqa_cases():
    """The reference's own GQA test grid (``tests/test_attention.py:43-54`` there)."""
    for dn, dt in DTYPES.items():
        for hd in (64, 128):
            for hq, hkv in ((8, 2), (8, 8), (4, 1)):
                for causal in (False, True):
                    yield f"gqa_{dn}_d{hd}_h{hq}_{hkv}_{'c' if causal else 'n'}", dt, hd, hq, hkv, causal


def gqa_inputs(dtype, head_dim, hq, hkv, seq_len=100):
    torch.manual_seed(0)
    q = torch.randn(1, hq, seq_len, head_dim, dtype=dtype)
    k = torch.randn(1, hkv, seq_len, head_dim, dtype=dtype)
    v = torch.randn(1, hkv, seq_len, head_dim, dtype=dtype)
    return q, k, v
