"""Host-side mirror of the reference's Python entry points for the decode path.

Signatures follow the reference binding (module ``fused_online_softmax_cuda``,
``fused_softmax_binding.cpp`` in the reference project):

* ``paged_attention_forward(query, key_cache, value_cache, block_tables, context_lens,
  softmax_scale=None)``                                             binding ``:109-173``
* ``fp8_paged_attention_forward(query, key_cache_fp8, value_cache_fp8, k_scale, v_scale,
  block_tables, context_lens, softmax_scale=None)``                 binding ``:634-718``
* ``async_flash_decode(q, k, v, softmax_scale=None)``               binding ``:308-360``
* ``fused_gqa_forward(q, k, v, is_causal=True, softmax_scale=None)``  binding ``:246-302`` (the prefill
  that fills the cache the decode path reads)

and raise ``RuntimeError`` with the reference's messages where the reference's ``TORCH_CHECK``s
fire.  Capabilities the reference does not have (GQA at decode, per-token / microscaling
scales, page sizes 32 and 64, q_len > 1, returned log-sum-exp) are keyword-only extensions.
All compute happens in libcuda_llm_b200.so; torch supplies device memory and the stream.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib as L

_DTYPE = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}
_workspaces = {}


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def get_workspace(device, nbytes: int) -> torch.Tensor:
    """A zero-initialised, per-(device, stream) scratch buffer that only grows."""
    key = (torch.device(device).index, _stream_ptr(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        L.check(L.load().cuda_llm_workspace_init(ws.data_ptr(), ws.numel(), _stream_ptr(device)),
                "cuda_llm_workspace_init")
        _workspaces[key] = ws
    return ws


_scratch_buffers = {}


def _scratch(device, nbytes: int, tag: str) -> torch.Tensor:
    """A per-(device, stream, tag) buffer that only grows, for temporaries that are not decode workspaces
    (those carry a status header and come from ``get_workspace``)."""
    key = (torch.device(device).index, _stream_ptr(device), tag)
    buf = _scratch_buffers.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _scratch_buffers[key] = buf
    return buf


def _scale_mode(k_scale: torch.Tensor) -> int:
    if k_scale.dtype in (torch.uint8, getattr(torch, "float8_e8m0fnu", torch.uint8)):
        if k_scale.dim() != 4:
            raise RuntimeError("E8M0 scales must be 4D [num_blocks, num_kv_heads, head_dim/32, page_size]")
        return L.SCALE_MX_E8M0
    if k_scale.dim() == 1:
        return L.SCALE_PER_HEAD
    if k_scale.dim() == 2:
        return L.SCALE_PER_BLOCK       # reference: per_block_scales = (k_scale.dim() == 2)
    if k_scale.dim() == 3:
        return L.SCALE_PER_TOKEN
    raise RuntimeError("Scale tensors must be 1D [heads], 2D [blocks, heads], 3D [blocks, heads, page] "
                       "or 4D E8M0 [blocks, heads, head_dim/32, page]")


def _byte_cache_format(key_cache, value_cache, kv_format: Optional[str]) -> int:
    """Element format of an 8-bit cache.  ``uint8`` / ``float8_e4m3fn`` bytes are E4M3 codes.  An
    ``int8`` tensor keeps the reference's integer meaning (``fp8_paged_attention_kernel.cuh:102`` in
    the reference project) unless ``kv_format='fp8_e4m3'`` states otherwise; the library has no
    integer reading and refuses it rather than reinterpret the bytes silently."""
    byte_types = (torch.int8, torch.uint8, torch.float8_e4m3fn)
    if key_cache.dtype not in byte_types or value_cache.dtype not in byte_types:
        raise RuntimeError("KV caches must be 8-bit quantized (int8 or uint8)")
    if kv_format not in (None, "fp8_e4m3"):
        raise RuntimeError(f"unknown kv_format {kv_format!r}: only 'fp8_e4m3' is provided")
    if kv_format is None and torch.int8 in (key_cache.dtype, value_cache.dtype):
        raise RuntimeError(
            "int8 KV caches are not accepted: this library reads cache bytes as FP8-E4M3 codes, the reference "
            "kernel reads them as integers (fp8_paged_attention_kernel.cuh:102). Pass uint8 / float8_e4m3fn "
            "tensors, or kv_format='fp8_e4m3' if the int8 tensor holds E4M3 codes.")
    return L.KV_FP8_E4M3


def fp8_paged_attention_forward(query, key_cache_fp8, value_cache_fp8, k_scale, v_scale,
                                block_tables, context_lens, softmax_scale=None, *,
                                cu_q_lens: Optional[torch.Tensor] = None, max_q_len: int = 1,
                                return_lse: bool = False, out: Optional[torch.Tensor] = None,
                                workspace: Optional[torch.Tensor] = None, num_ctas: int = 0,
                                check_status: bool = False, flags: int = 0,
                                kv_format: Optional[str] = None, split_context=None,
                                rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
                                rope_positions: Optional[torch.Tensor] = None):
    """Decode attention over a paged FP8 / MXFP8 / MXFP4 KV cache.

    query ``[total_q, Hq, D]``; caches ``[num_blocks, Hkv, D, page]`` bytes (V may be packed
    E2M1 ``[num_blocks, Hkv, D/2, page]`` with E8M0 scales); ``Hkv = cache.shape[1]`` may be
    smaller than ``Hq`` (GQA: kv_head = q_head // (Hq // Hkv), the rule of
    ``fused_gqa_kernel.cuh:39-41`` in the reference project).  Bytes are E4M3 codes: this is
    the semantics the reference's own test specifies (``tests/test_kernels_misc.py:42-64``),
    not the int8 cast its kernel performs (``fp8_paged_attention_kernel.cuh:102``).  A
    ``torch.uint8`` or ``torch.float8_e4m3fn`` cache is read that way; a ``torch.int8`` cache is
    refused unless ``kv_format="fp8_e4m3"`` says that its bytes are E4M3 codes too, because a caller
    of the reference with real int8 data would otherwise get different numbers without a word.

    ``rope_cos`` / ``rope_sin`` (fp32 ``[positions, D]``, the tables of the reference's
    ``tests/_utils.py:75-81``): the query is rotated (rotate-half convention,
    ``fused_rope_flash_attention_kernel.cuh:56-74`` in the reference project) as it is loaded, at
    ``rope_positions`` (int32 ``[total_q]``) or, by default, at ``context_len - q_len + j``.

    ``split_context=(nccl_comm_ptr, nranks, rank, exchange)``: the cache, tables and lengths describe
    this rank's KV range of a context sharded over ``nranks`` GPUs; the call then runs the local
    decode, one NCCL all-gather of the fp32 (out | lse) blocks and the merge from a single C++ entry
    point (``cuda_llm_split_context_decode``) and returns the merged result on every rank.
    ``exchange`` is a uint8 CUDA tensor of ``cuda_llm_split_context_exchange_bytes`` bytes.
    """
    if not (query.is_cuda and key_cache_fp8.is_cuda and value_cache_fp8.is_cuda):
        raise RuntimeError("Inputs must be on CUDA")
    if not (k_scale.is_cuda and v_scale.is_cuda):
        raise RuntimeError("Scale tensors must be on CUDA")
    if not (block_tables.is_cuda and context_lens.is_cuda):
        raise RuntimeError("Metadata tensors must be on CUDA")
    if query.dim() != 3:
        raise RuntimeError("Query must be 3D [num_seqs, num_heads, head_dim]")
    if key_cache_fp8.dim() != 4 or value_cache_fp8.dim() != 4:
        raise RuntimeError("KV caches must be 4D [num_blocks, num_heads, head_dim, page_size]")
    k_format = _byte_cache_format(key_cache_fp8, value_cache_fp8, kv_format)
    if query.dtype not in _DTYPE:
        raise RuntimeError("Unsupported query scalar type for FP8 PagedAttention. "
                           "Supported: Float32, Float16, BFloat16.")
    total_q, hq, d = query.shape
    nb, hkv, dk, page = key_cache_fp8.shape
    if d not in (64, 128):
        raise RuntimeError("Only head_dim 64 and 128 supported")
    if page not in (16, 32, 64):
        raise RuntimeError("Only page_size 16, 32 and 64 are supported")
    if dk != d:
        raise RuntimeError("key cache head_dim does not match the query")
    if value_cache_fp8.shape[2] == d:
        v_format = L.KV_FP8_E4M3
    elif value_cache_fp8.shape[2] * 2 == d:
        v_format = L.KV_FP4_E2M1
    else:
        raise RuntimeError("value cache head_dim does not match the query")
    if hq % hkv:
        raise RuntimeError("num_heads must be a multiple of the cache's num_kv_heads")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise RuntimeError("block_tables and context_lens must be int32")
    num_seqs = context_lens.shape[0]
    if cu_q_lens is None and total_q != num_seqs:
        raise RuntimeError("query has more rows than sequences: pass cu_q_lens")
    for t, name in ((query, "query"), (key_cache_fp8, "key_cache"), (value_cache_fp8, "value_cache"),
                    (block_tables, "block_tables"), (context_lens, "context_lens")):
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    mode = _scale_mode(k_scale)
    if mode != L.SCALE_MX_E8M0:
        # the reference converts scales to fp32 contiguous temporaries (binding :680-681)
        k_scale = k_scale.to(torch.float32).contiguous()
        v_scale = v_scale.to(torch.float32).contiguous()
    else:
        k_scale = k_scale.contiguous()
        v_scale = v_scale.contiguous()
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)

    lib = L.load()
    with torch.cuda.device(query.device):
        if out is None:
            out = torch.empty_like(query)                        # reference: empty_like(query)
        lse = torch.empty(total_q, hq, dtype=torch.float32, device=query.device) if return_lse else None
        need = lib.cuda_llm_paged_decode_workspace_bytes(num_seqs, hq, hkv, d, page, max_q_len, num_ctas)
        if need == 0:
            raise L.CudaLlmError(L.EINVAL, "cuda_llm_paged_decode_workspace_bytes")
        ws = workspace if workspace is not None else get_workspace(query.device, need)
        p = L.PagedDecodeParams(
            query=query.data_ptr(), key_cache=key_cache_fp8.data_ptr(),
            value_cache=value_cache_fp8.data_ptr(), k_scale=k_scale.data_ptr(),
            v_scale=v_scale.data_ptr(), block_tables=block_tables.data_ptr(),
            context_lens=context_lens.data_ptr(), cu_q_lens=_ptr(cu_q_lens), out=out.data_ptr(),
            lse=_ptr(lse), workspace=ws.data_ptr(), workspace_bytes=ws.numel(),
            num_seqs=num_seqs, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page,
            max_blocks_per_seq=block_tables.shape[1], num_blocks=nb, max_q_len=max_q_len,
            q_dtype=_DTYPE[query.dtype], out_dtype=_DTYPE[out.dtype], k_format=k_format,
            v_format=v_format, scale_mode=mode, softmax_scale=scale, num_ctas=num_ctas, flags=flags)
        if rope_cos is not None:
            if rope_sin is None or rope_cos.shape != rope_sin.shape or rope_cos.dim() != 2 or rope_cos.shape[1] != d:
                raise RuntimeError("rope_cos / rope_sin must both be [positions, head_dim]")
            rope_cos = rope_cos.to(device=query.device, dtype=torch.float32).contiguous()
            rope_sin = rope_sin.to(device=query.device, dtype=torch.float32).contiguous()
            if rope_positions is not None:
                rope_positions = rope_positions.to(device=query.device, dtype=torch.int32).contiguous()
            p.rope_cos, p.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
            p.rope_positions, p.rope_num_positions = _ptr(rope_positions), rope_cos.shape[0]
        if split_context is not None:
            comm, nranks, rank, exch = split_context
            L.check(lib.cuda_llm_split_context_decode(C.byref(p), comm, nranks, rank, exch.data_ptr(), exch.numel(),
                                                      _stream_ptr(query.device)), "cuda_llm_split_context_decode")
        else:
            L.check(lib.cuda_llm_paged_decode(C.byref(p), _stream_ptr(query.device)), "cuda_llm_paged_decode")
        if check_status:
            st = decode_status(ws, query.device)
            if st:
                raise RuntimeError(f"paged decode reported device status 0x{st:x}")
    return (out, lse) if return_lse else out


def nccl_comm_ptr(group=None, device=None) -> int:
    """The ncclComm_t torch.distributed uses for ``group`` on ``device`` (an integer address), for
    ``split_context=``.  The communicator exists once the group has run a collective on that device."""
    import torch.distributed as dist
    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(pg._get_backend(dev)._comm_ptr())


def split_context_exchange(rows: int, head_dim: int, nranks: int, device) -> torch.Tensor:
    """The exchange buffer of the split-context mode: ``nranks`` blocks of fp32 out [rows, D] + lse [rows]."""
    n = L.load().cuda_llm_split_context_exchange_bytes(rows, head_dim, nranks)
    return torch.empty(n, dtype=torch.uint8, device=device)


def paged_attention_forward(query, key_cache, value_cache, block_tables, context_lens, softmax_scale=None, *,
                            cu_q_lens: Optional[torch.Tensor] = None, max_q_len: int = 1,
                            return_lse: bool = False, num_ctas: int = 0, check_status: bool = False,
                            flags: int = 0):
    """Decode attention over a paged fp32 / fp16 / bf16 cache: signature of the reference binding
    ``paged_attention_forward`` (``fused_softmax_binding.cpp:109-173`` in the reference project).
    ``key_cache.shape[1]`` may be smaller than ``query.shape[1]`` (GQA).  The keyword-only extensions
    (several query rows per sequence, log-sum-exp output) exist for a 16-bit cache only."""
    if not (query.is_cuda and key_cache.is_cuda and value_cache.is_cuda):
        raise RuntimeError("Inputs must be on CUDA")
    if not (block_tables.is_cuda and context_lens.is_cuda):
        raise RuntimeError("Metadata tensors must be on CUDA")
    if query.dim() != 3:
        raise RuntimeError("Query must be 3D [num_seqs, num_heads, head_dim]")
    if key_cache.dim() != 4 or value_cache.dim() != 4:
        raise RuntimeError("KV caches must be 4D [num_blocks, num_heads, head_dim, page_size]")
    if query.dtype not in _DTYPE:
        raise RuntimeError("Unsupported scalar type for PagedAttention. Supported: Float32, Float16, BFloat16.")
    if key_cache.dtype != query.dtype or value_cache.dtype != query.dtype:
        raise RuntimeError("query and KV caches must have the same dtype")
    n, hq, d = query.shape
    nb, hkv, dk, page = key_cache.shape
    if d not in (64, 128) or dk != d:
        raise RuntimeError("Only head_dim 64 and 128 supported")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise RuntimeError("block_tables and context_lens must be int32")
    for t, name in ((query, "query"), (key_cache, "key_cache"), (value_cache, "value_cache"),
                    (block_tables, "block_tables"), (context_lens, "context_lens")):
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    lib = L.load()
    extended = cu_q_lens is not None or return_lse or num_ctas or check_status or flags
    if extended:
        if query.dtype == torch.float32:
            raise RuntimeError("cu_q_lens / return_lse need a float16 or bfloat16 cache")
        if page not in (16, 32, 64):
            raise RuntimeError("Only page_size 16, 32 and 64 are supported")
        num_seqs = context_lens.shape[0]
        fmt = L.KV_F16 if query.dtype == torch.float16 else L.KV_BF16
        with torch.cuda.device(query.device):
            out = torch.empty_like(query)
            lse = torch.empty(n, hq, dtype=torch.float32, device=query.device) if return_lse else None
            need = lib.cuda_llm_paged_decode_workspace_bytes(num_seqs, hq, hkv, d, page, max_q_len, num_ctas)
            if need == 0:
                raise L.CudaLlmError(L.EINVAL, "cuda_llm_paged_decode_workspace_bytes")
            ws = get_workspace(query.device, need)
            p = L.PagedDecodeParams(
                query=query.data_ptr(), key_cache=key_cache.data_ptr(), value_cache=value_cache.data_ptr(),
                k_scale=None, v_scale=None, block_tables=block_tables.data_ptr(),
                context_lens=context_lens.data_ptr(), cu_q_lens=_ptr(cu_q_lens), out=out.data_ptr(),
                lse=_ptr(lse), workspace=ws.data_ptr(), workspace_bytes=ws.numel(),
                num_seqs=num_seqs, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page,
                max_blocks_per_seq=block_tables.shape[1], num_blocks=nb, max_q_len=max_q_len,
                q_dtype=_DTYPE[query.dtype], out_dtype=_DTYPE[out.dtype], k_format=fmt, v_format=fmt,
                scale_mode=0, softmax_scale=scale, num_ctas=num_ctas, flags=flags)
            L.check(lib.cuda_llm_paged_decode(C.byref(p), _stream_ptr(query.device)), "cuda_llm_paged_decode")
            if check_status:
                st = decode_status(ws, query.device)
                if st:
                    raise RuntimeError(f"paged decode reported device status 0x{st:x}")
        return (out, lse) if return_lse else out
    with torch.cuda.device(query.device):
        out = torch.empty_like(query)
        need = lib.cuda_llm_dense_decode_workspace_bytes(n, hq, hkv, d, block_tables.shape[1] * page)
        if need == 0:
            raise L.CudaLlmError(L.EINVAL, "cuda_llm_dense_decode_workspace_bytes")
        ws = get_workspace(query.device, need)
        L.check(lib.cuda_llm_paged_attention(query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                                             block_tables.data_ptr(), context_lens.data_ptr(), out.data_ptr(),
                                             n, hq, hkv, d, page, block_tables.shape[1], nb, scale,
                                             _DTYPE[query.dtype], ws.data_ptr(), ws.numel(),
                                             _stream_ptr(query.device)), "cuda_llm_paged_attention")
    return out


def async_flash_decode(q, k, v, softmax_scale=None):
    """Decode attention over contiguous KV: signature of the reference binding ``async_flash_decode``
    (``fused_softmax_binding.cpp:308-360``): q [B,H,1,D], k/v [B,Hkv,S,D] -> [B,H,1,D]."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("Inputs must be on CUDA")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("Inputs must be 4D [batch, heads, seq, dim]")
    if q.size(2) != 1:
        raise RuntimeError("Query sequence length must be 1 for Flash-Decoding")
    if k.shape != v.shape:
        raise RuntimeError("K and V must have identical shapes")
    if q.dtype not in _DTYPE:
        raise RuntimeError("Unsupported scalar type for Async Flash-Decode. Supported: Float32, Float16, BFloat16.")
    b, h, _, d = q.shape
    if d not in (64, 128):
        raise RuntimeError("Only head_dim 64 and 128 supported")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    hkv, s = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    lib = L.load()
    with torch.cuda.device(q.device):
        out = torch.empty_like(q)
        need = lib.cuda_llm_dense_decode_workspace_bytes(b, h, hkv, d, s)
        if need == 0:
            raise L.CudaLlmError(L.EINVAL, "cuda_llm_dense_decode_workspace_bytes")
        ws = get_workspace(q.device, need)
        L.check(lib.cuda_llm_flash_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, h, hkv, s, d,
                                          scale, _DTYPE[q.dtype], ws.data_ptr(), ws.numel(),
                                          _stream_ptr(q.device)), "cuda_llm_flash_decode")
    return out


def fused_gqa_forward(q, k, v, is_causal=True, softmax_scale=None, *, paged_kv=None):
    """Grouped-query attention over a whole prompt: signature of the reference binding
    ``fused_gqa_forward`` (``fused_softmax_binding.cpp:246-302``, ``m.def`` ``:751-756`` in the
    reference project): q ``[B, Hq, S, D]``, k / v ``[B, Hkv, S, D]`` -> ``[B, Hq, S, D]``.

    ``paged_kv=(key_cache, value_cache, k_scale, v_scale, slot_block, slot_offset)``: the same call
    also quantises K / V into the paged cache (formats inferred from the tensors as in
    ``fp8_paged_attention_forward``; ``slot_block`` / ``slot_offset`` int32 ``[B * S]``), so that the
    prompt's KV is ready for the decode entry points."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("Inputs must be on CUDA")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("Inputs must be 4D [batch, heads, seq, dim]")
    if k.shape != v.shape:
        raise RuntimeError("K and V must have identical shapes")
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    if hq % hkv:
        raise RuntimeError("num_q_heads must be divisible by num_kv_heads")
    if d not in (64, 128):
        raise RuntimeError("Only head_dim 64 and 128 supported")
    if q.dtype not in _DTYPE:
        raise RuntimeError("Unsupported scalar type for GQA. Supported: Float32, Float16, BFloat16.")
    if k.dtype != q.dtype or v.dtype != q.dtype or k.shape[0] != b or k.shape[2] != s or k.shape[3] != d:
        raise RuntimeError("q, k and v must share dtype, batch, sequence length and head_dim")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    target = None
    if paged_kv is not None:
        kc, vc, ks, vs, slot_block, slot_offset = paged_kv
        mode = _scale_mode(ks)
        v_format = L.KV_FP8_E4M3 if vc.shape[2] == d else L.KV_FP4_E2M1
        slot_block = slot_block.to(device=q.device, dtype=torch.int32).contiguous()
        slot_offset = slot_offset.to(device=q.device, dtype=torch.int32).contiguous()
        if slot_block.numel() != b * s or slot_offset.numel() != b * s:
            raise RuntimeError("slot_block / slot_offset need one entry per (batch, position)")
        target = L.KvCacheTarget(key_cache=kc.data_ptr(), value_cache=vc.data_ptr(), k_scale=ks.data_ptr(),
                                 v_scale=vs.data_ptr(), slot_block=slot_block.data_ptr(),
                                 slot_offset=slot_offset.data_ptr(), status=None, page_size=kc.shape[3],
                                 num_blocks=kc.shape[0], v_format=v_format, scale_mode=mode)
    with torch.cuda.device(q.device):
        out = torch.empty_like(q)
        L.check(L.load().cuda_llm_gqa_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, hq, hkv, s, d,
                                              scale, 1 if is_causal else 0, _DTYPE[q.dtype],
                                              C.byref(target) if target is not None else None,
                                              _stream_ptr(q.device)), "cuda_llm_gqa_prefill")
    return out


def fused_microscaled_attention(q, q_scale, k, k_scale, v, v_scale, is_causal=True, softmax_scale=None, *,
                                out_dtype=torch.bfloat16):
    """Dense attention over microscaled FP8 tensors (the reference declares
    ``dispatch_fused_microscaled_attention``, ``kernels_api.h:103-108`` in the reference project,
    without a definition or a binding): q ``[B, Hq, S, D]``, k / v ``[B, Hkv, S, D]`` E4M3 codes
    (uint8 / float8_e4m3fn), ``*_scale [B, H, S, D/32]`` fp32, one per 32 elements of head_dim."""
    for t_ in (q, k, v, q_scale, k_scale, v_scale):
        if not t_.is_cuda:
            raise RuntimeError("Inputs must be on CUDA")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("Inputs must be 4D [batch, heads, seq, dim]")
    if k.shape != v.shape:
        raise RuntimeError("K and V must have identical shapes")
    for t_ in (q, k, v):
        if t_.dtype not in (torch.uint8, torch.float8_e4m3fn):
            raise RuntimeError("q, k and v must hold E4M3 codes (uint8 or float8_e4m3fn)")
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    if hq % hkv:
        raise RuntimeError("num_q_heads must be divisible by num_kv_heads")
    if d not in (64, 128):
        raise RuntimeError("Only head_dim 64 and 128 supported")
    if tuple(q_scale.shape) != (b, hq, s, d // 32) or tuple(k_scale.shape) != (b, hkv, s, d // 32) \
            or tuple(v_scale.shape) != (b, hkv, s, d // 32):
        raise RuntimeError("scales must be [batch, heads, seq, head_dim/32]")
    if out_dtype not in _DTYPE:
        raise RuntimeError("Unsupported output scalar type. Supported: Float32, Float16, BFloat16.")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    qs, ks, vs = (x.to(torch.float32).contiguous() for x in (q_scale, k_scale, v_scale))
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    with torch.cuda.device(q.device):
        out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
        lib = L.load()
        need = lib.cuda_llm_mx_attention_workspace_bytes(b, hq, hkv, s, d)   # 0: no tcgen05 route for this shape
        ws = _scratch(q.device, need, "mx_attention") if need else None
        L.check(lib.cuda_llm_mx_attention_ws(q.data_ptr(), qs.data_ptr(), k.data_ptr(), ks.data_ptr(), v.data_ptr(),
                                             vs.data_ptr(), out.data_ptr(), b, hq, hkv, s, d, scale,
                                             1 if is_causal else 0, _DTYPE[out_dtype],
                                             ws.data_ptr() if need else None, ws.numel() if need else 0,
                                             _stream_ptr(q.device)),
                "cuda_llm_mx_attention_ws")
    return out


flash_decode = async_flash_decode      # the name the reference's README gives the Python-level call


def kv_cache_append(k_new, v_new, slot_block, slot_offset, key_cache, value_cache, k_scale, v_scale):
    """Quantise and store new K/V tokens ``[n, Hkv, D]`` at pages ``slot_block`` / offsets
    ``slot_offset`` (int32 ``[n]``).  Scale mode and V format are taken from the cache tensors as in
    ``fp8_paged_attention_forward``; per-token and E8M0 scales are written, coarser scales are read."""
    n, hkv, d = k_new.shape
    nb, _, _, page = key_cache.shape
    mode = _scale_mode(k_scale)
    v_format = L.KV_FP8_E4M3 if value_cache.shape[2] == d else L.KV_FP4_E2M1
    if k_new.dtype not in _DTYPE or v_new.dtype != k_new.dtype:
        raise RuntimeError("new K/V must be float32, float16 or bfloat16 and of one dtype")
    k_new, v_new = k_new.contiguous(), v_new.contiguous()
    with torch.cuda.device(k_new.device):
        L.check(L.load().cuda_llm_kv_append(k_new.data_ptr(), v_new.data_ptr(), slot_block.data_ptr(),
                                            slot_offset.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                                            k_scale.data_ptr(), v_scale.data_ptr(), n, hkv, d, page, nb,
                                            _DTYPE[k_new.dtype], v_format, mode, None,
                                            _stream_ptr(k_new.device)), "cuda_llm_kv_append")


def decode_status(workspace: torch.Tensor, device=None) -> int:
    """Read and clear the device status word (synchronises the current stream)."""
    device = workspace.device if device is None else device
    st = C.c_uint32(0)
    L.check(L.load().cuda_llm_decode_status(workspace.data_ptr(), _stream_ptr(device), C.byref(st)),
            "cuda_llm_decode_status")
    return int(st.value)


def merge_partials(parts_out: torch.Tensor, parts_lse: torch.Tensor, out_dtype=torch.float32,
                   return_lse: bool = False):
    """parts_out [P, ..., D] fp32, parts_lse [P, ...] -> merged [..., D] (and lse [...])."""
    if not parts_out.is_cuda:
        raise RuntimeError("Inputs must be on CUDA")
    parts_out = parts_out.contiguous().float()
    parts_lse = parts_lse.contiguous().float()
    P, d = parts_out.shape[0], parts_out.shape[-1]
    rows = parts_lse[0].numel()
    with torch.cuda.device(parts_out.device):
        out = torch.empty(parts_out.shape[1:], dtype=out_dtype, device=parts_out.device)
        lse = torch.empty(parts_lse.shape[1:], dtype=torch.float32, device=parts_out.device) if return_lse else None
        L.check(L.load().cuda_llm_merge_partials(parts_out.data_ptr(), parts_lse.data_ptr(), P, rows, d,
                                                 out.data_ptr(), _DTYPE[out_dtype], _ptr(lse),
                                                 _stream_ptr(parts_out.device)), "cuda_llm_merge_partials")
    return (out, lse) if return_lse else out


def dequant_pages(cache: torch.Tensor, scale: torch.Tensor, pages: torch.Tensor, head_dim: int,
                  fmt: int, scale_mode: int) -> torch.Tensor:
    """fp32 [n, Hkv, D, page] of the listed pages (bit-exact decode of the stored codes)."""
    nb, hkv, _, page = cache.shape
    pages = pages.to(torch.int32).contiguous()
    with torch.cuda.device(cache.device):
        out = torch.empty(pages.numel(), hkv, head_dim, page, dtype=torch.float32, device=cache.device)
        L.check(L.load().cuda_llm_dequant_pages(cache.data_ptr(), scale.data_ptr(), pages.data_ptr(),
                                                pages.numel(), hkv, head_dim, page, fmt, scale_mode,
                                                out.data_ptr(), _stream_ptr(cache.device)),
                "cuda_llm_dequant_pages")
    return out


_FMT = {"fp8_e4m3": L.KV_FP8_E4M3, "fp4_e2m1": L.KV_FP4_E2M1}
_MODE = {"per_head": L.SCALE_PER_HEAD, "per_block": L.SCALE_PER_BLOCK, "per_token": L.SCALE_PER_TOKEN,
         "mx_e8m0": L.SCALE_MX_E8M0}


def run_workload(wl, *, return_lse=False, out=None, num_ctas=0, check_status=False, workspace=None,
                 flags=0, split_context=None):
    """Run a ``workloads.DecodeWorkload`` through ``fp8_paged_attention_forward``."""
    return fp8_paged_attention_forward(
        wl.query, wl.key_cache, wl.value_cache, wl.k_scale, wl.v_scale, wl.block_tables,
        wl.context_lens, wl.softmax_scale, cu_q_lens=wl.cu_q_lens, max_q_len=wl.max_q_len,
        return_lse=return_lse, out=out, num_ctas=num_ctas, check_status=check_status,
        workspace=workspace, flags=flags, split_context=split_context)
