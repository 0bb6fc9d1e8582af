"""The REAL reference kernel (compiled from the reference's sources into oracle/_ref by
oracle/Makefile) on the reference's own paged cases: it must agree with the golden outputs of its
Python specification and with this library's paged_attention.  Skipped when oracle/_ref was not
built (the reference checkout is not present on every machine)."""
import ctypes as C
import os

import pytest
import torch

import cases
from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_paged.so")


@pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref not built")
@pytest.mark.parametrize("case", list(cases.paged_cases()), ids=lambda c: c[0])
def test_reference_cuda_kernel_vs_golden_and_ours(golden, case):
    from cuda_b200 import ops
    ref = C.CDLL(REF)
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc, vc = O.paged_layout_from_dense(k, 16, perm).cuda(), O.paged_layout_from_dense(v, 16, perm).cuda()
    qd, btd, ld = q.cuda(), bt.cuda(), lens_t.cuda()
    out_ref = torch.empty_like(qd)
    rc = ref.ref_paged_attention(C.c_void_p(qd.data_ptr()), C.c_void_p(kc.data_ptr()), C.c_void_p(vc.data_ptr()),
                                 C.c_void_p(btd.data_ptr()), C.c_void_p(ld.data_ptr()), C.c_void_p(out_ref.data_ptr()),
                                 3, 4, hd, bt.shape[1], C.c_float(1.0 / hd ** 0.5),
                                 1 if dtype == torch.float16 else 2, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0
    gold = torch.from_numpy(golden[f"{name}/out"])
    atol, rtol = (2e-2, 2e-2) if dtype == torch.float16 else (4e-2, 4e-2)
    assert torch.allclose(out_ref.float().cpu(), gold, atol=atol, rtol=rtol)
    ours = ops.paged_attention_forward(qd, kc, vc, btd, ld)
    assert torch.allclose(ours.float(), out_ref.float(), atol=atol, rtol=rtol)
