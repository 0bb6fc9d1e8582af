"""The reference's own binding TU (fused_softmax_binding.cpp, compiled unchanged with the three decode
entry points and the GQA prefill switched on) linked against libcuda_llm_b200.so: its Python functions replay the
reference's test cases on this library's kernels.  Built by `make -C oracle refbinding` where the
reference checkout is mounted; the test is skipped where that build is absent.  Runs in a child
process because the module carries the same name as this repository's own extension."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFBIND = os.path.join(ROOT, "oracle", "_ref", "refbinding")

CHILD = r'''
import sys
import numpy as np
import torch
sys.path[:0] = [REFBIND, ROOT, ROOT + "/tests", ROOT + "/tests/golden"]
import fused_online_softmax_cuda as ext
assert ext.__file__.startswith(REFBIND), ext.__file__
import cases
from oracle import paged_decode_oracle as O
golden = np.load(ROOT + "/tests/golden/reference_cases.npz")
TOL = {torch.float32: (1e-4, 1e-4), torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2)}
n = 0
for name, dtype, hd, lens in cases.paged_cases():
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc, vc = O.paged_layout_from_dense(k, 16, perm).cuda(), O.paged_layout_from_dense(v, 16, perm).cuda()
    out = ext.paged_attention_forward(q.cuda(), kc, vc, bt.cuda(), lens_t.cuda())
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=TOL[dtype][0], rtol=TOL[dtype][1]), name
    n += 1
for name, dtype, hd, lens in cases.fp8_cases():
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    k8, v8, ks, vs, _, _ = cases.fp8_quantise(k, v)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc, vc = O.paged_layout_from_dense(k8, 16, perm).cuda(), O.paged_layout_from_dense(v8, 16, perm).cuda()
    out = ext.fp8_paged_attention_forward(q.cuda(), kc, vc, ks.cuda(), vs.cuda(), bt.cuda(), lens_t.cuda())
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=TOL[dtype][0], rtol=TOL[dtype][1]), name
    n += 1
for name, dtype, hd, kv_len in cases.decode_cases():
    q, k, v = cases.decode_inputs(dtype, hd, kv_len)
    out = ext.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=TOL[dtype][0], rtol=TOL[dtype][1]), name
    n += 1
for name, dtype, hd, hq, hkv, causal in cases.gqa_cases():
    q, k, v = cases.gqa_inputs(dtype, hd, hq, hkv)
    out = ext.fused_gqa_forward(q.cuda(), k.cuda(), v.cuda(), is_causal=causal)
    rows = torch.from_numpy(golden[f"{name}/rows"])
    assert torch.allclose(out[:, :, list(cases.GQA_ROWS), :].float().cpu(), rows, atol=TOL[dtype][0], rtol=TOL[dtype][1]), name
    n += 1
print("REFERENCE BINDING OK", n)
'''


@pytest.mark.skipif(not os.path.exists(os.path.join(REFBIND, "fused_online_softmax_cuda.so")),
                    reason="oracle/_ref/refbinding not built (needs the reference checkout)")
def test_reference_binding_runs_on_this_library():
    code = f"REFBIND = {REFBIND!r}\nROOT = {ROOT!r}\n" + CHILD
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "REFERENCE BINDING OK" in r.stdout
