"""Generate golden vectors by running the REFERENCE's own specification functions.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's ``tests/_utils.py`` (``make_paged_cache``, ``ref_decode``,
``ref_attention``) and replays the reference's own test cases
(``tests/test_kernels_misc.py:26-35`` paged, ``:42-64`` E4M3 paged,
``tests/test_attention.py:76-86`` decode, ``ref_rope_attention`` of ``tests/_utils.py:91-93`` for the
rotary case, ``ref_gqa`` ``:67-72`` on the grid of ``tests/test_attention.py:43-54`` for the prefill) on the CPU with the same seed rule
(``tests/conftest.py:31-33``: ``torch.manual_seed(0)`` before every case).  Inputs are
regenerated from the seed by ``tests/golden/cases.py`` at test time; the fixture keeps the
reference outputs, the block tables the reference drew, and CRC32s of the paged caches so
the tests can prove that the inputs and the page layout are bit-identical.
"""
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def crc(t: torch.Tensor) -> int:
    return zlib.crc32(t.contiguous().view(torch.uint8).numpy().tobytes())


def main(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import _utils as ref  # the reference's specification module

    out = {}
    # ---- paged attention, fp16 / bf16 caches --------------------------------------------
    for name, dtype, head_dim, lens in cases.paged_cases():
        q, k, v, lens_t = cases.paged_inputs(dtype, head_dim, lens)
        kc, vc, bt = ref.make_paged_cache(k, v, cases.PAGE)
        o = ref.ref_decode(q, k, v, lens_t)
        out[f"{name}/bt"] = bt.numpy()
        out[f"{name}/out"] = o.numpy()
        out[f"{name}/crc"] = np.array([crc(q), crc(kc), crc(vc)], dtype=np.uint32)
    # ---- E4M3 paged attention, per-head scales ------------------------------------------
    for name, dtype, head_dim, lens in cases.fp8_cases():
        q, k, v, lens_t = cases.paged_inputs(dtype, head_dim, lens)
        k8, v8, ks, vs, k_deq, v_deq = cases.fp8_quantise(k, v)
        kc, vc, bt = ref.make_paged_cache(k8, v8, cases.PAGE)
        o = ref.ref_decode(q, k_deq, v_deq, lens_t)
        out[f"{name}/bt"] = bt.numpy()
        out[f"{name}/out"] = o.numpy()
        out[f"{name}/crc"] = np.array([crc(q), crc(kc), crc(vc), crc(ks), crc(vs)], dtype=np.uint32)
    # ---- contiguous decode ---------------------------------------------------------------
    for name, dtype, head_dim, kv_len in cases.decode_cases():
        q, k, v = cases.decode_inputs(dtype, head_dim, kv_len)
        o = ref.ref_attention(q, k, v)
        out[f"{name}/out"] = o.numpy()
        out[f"{name}/crc"] = np.array([crc(q), crc(k), crc(v)], dtype=np.uint32)
    # ---- GQA convention (ref_gqa) on a decode-shaped case --------------------------------
    torch.manual_seed(0)
    q = torch.randn(2, 8, 1, 64)
    k = torch.randn(2, 2, 77, 64)
    v = torch.randn(2, 2, 77, 64)
    out["gqa_decode/out"] = ref.ref_gqa(q, k, v, is_causal=False).numpy()
    out["gqa_decode/crc"] = np.array([crc(q), crc(k), crc(v)], dtype=np.uint32)

    # ---- rotary embedding: last row of the reference's causal RoPE attention = one decode step ----
    for name, dtype, head_dim, seq_len in cases.rope_cases():
        q, k, v = cases.rope_inputs(dtype, head_dim, seq_len)
        cos, sin = ref.rope_tables(seq_len, head_dim, "cpu")
        o = ref.ref_rope_attention(q, k, v, cos, sin, is_causal=True)
        out[f"{name}/out_last"] = o[:, :, -1, :].contiguous().numpy()          # [B, H, D]
        k_rot = ref.apply_rope(k, cos, sin).to(dtype)                           # what the cache holds
        out[f"{name}/crc"] = np.array([crc(q), crc(k), crc(v), crc(cos), crc(sin), crc(k_rot)], dtype=np.uint32)

    # ---- GQA prefill: the reference's own test grid, sampled output rows --------------------------
    for name, dtype, head_dim, hq, hkv, causal in cases.gqa_cases():
        q, k, v = cases.gqa_inputs(dtype, head_dim, hq, hkv)
        o = ref.ref_gqa(q, k, v, is_causal=causal)                              # [1, Hq, S, D] fp32
        out[f"{name}/rows"] = o[:, :, list(cases.GQA_ROWS), :].contiguous().numpy()
        out[f"{name}/crc"] = np.array([crc(q), crc(k), crc(v), crc(o)], dtype=np.uint32)

    path = os.path.join(HERE, "reference_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays; torch", torch.__version__)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
