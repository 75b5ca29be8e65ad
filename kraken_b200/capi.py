"""ctypes binding of libkrk_cuda.so: one Python function per entry of include/krk_cuda.h.

This is glue, not a second implementation: every function checks nothing and computes
nothing itself, it passes device pointers (``tensor.data_ptr()``) and sizes to the C ABI
and raises ``KrkCudaError`` on a non-zero status. torch supplies device memory and streams.
If the library has not been built, importing this module raises: there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkrk_cuda.so")

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
Q5_0, Q5_1, Q5_K = 6, 7, 13
Q2_K, Q3_K, IQ4_NL = 10, 11, 20
X_F32, X_F16 = 0, 1
MAX_GROUP, MAX_ROWS = 16, 8


class KrkCudaError(RuntimeError):
    def __init__(self, rc: int, where: str):
        self.rc = rc
        detail = lib.krk_cuda_last_cuda_error().decode() if rc == -5 else ""
        super().__init__(f"{where}: {lib.krk_cuda_strerror(rc).decode()} (rc={rc}) {detail}".strip())


if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m kraken_b200.build` "
                      "(this package has no fallback path)")

lib = C.CDLL(LIB_PATH)

_vp, _i64, _int, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t


class GgufTensorInfo(C.Structure):
    """struct krk_gguf_tensor"""
    _fields_ = [("name", C.c_char_p), ("type_id", _int), ("supported", _int), ("n_dims", _int), ("ne", _i64 * 4),
                ("host_data", _vp), ("n_bytes", _sz)]


class ExpertBank(C.Structure):
    """struct krk_cuda_expert_bank"""
    _fields_ = [("gate", _vp), ("up", _vp), ("down", _vp), ("wt_gate_up", _int), ("wt_down", _int),
                ("n_local", _int), ("expert_base", _int), ("n_embd", _i64), ("n_ff", _i64)]


# name -> (restype, argtypes); the list tests/ checks against the header.
SIGNATURES = {
    "krk_cuda_strerror": (C.c_char_p, [_int]),
    "krk_cuda_last_cuda_error": (C.c_char_p, []),
    "krk_cuda_dtype_ok": (_int, [_int]),
    "krk_cuda_block_size": (_int, [_int]),
    "krk_cuda_block_bytes": (_int, [_int]),
    "krk_cuda_row_bytes": (_sz, [_int, _i64]),
    "krk_cuda_gemm_k_ok": (_int, [_int, _i64]),
    "krk_cuda_dequant_rows": (_int, [_vp, _vp, _int, _i64, _i64, _vp]),
    "krk_cuda_gemv": (_int, [_vp, _vp, _vp, _int, _i64, _i64, _i64, _int, _vp]),
    "krk_cuda_gemv_group": (_int, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_int),
                                   C.POINTER(_i64), _i64, _int, _int, _vp]),
    "krk_cuda_gemm_workspace_bytes": (_sz, [_int, _i64, _i64, _i64]),
    "krk_cuda_gemm": (_int, [_vp, _vp, _int, _vp, _int, _i64, _i64, _i64, _vp, _sz, _vp]),
    "krk_cuda_gemm_f32_static": (_int, [_vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    "krk_cuda_gemm_f32_static_status": (_int, []),
    "krk_cuda_route": (_int, [_vp, _vp, _vp, _i64, _int, _int, _vp]),
    "krk_cuda_router_softmax": (_int, [_vp, _vp, _i64, _int, _vp]),
    "krk_cuda_router_topk": (_int, [_vp, _i64, _int, _int, _vp, _vp, _int, C.c_float, _vp]),
    "krk_cuda_moe_plan_build": (_int, [_vp, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp]),
    "krk_cuda_shard_allgather": (_int, [_vp, _vp, _sz, _vp, _vp]),
    "krk_cuda_nccl_unique_id": (_int, [C.c_char_p]),
    "krk_cuda_nccl_comm_init": (_int, [C.POINTER(_vp), _int, _int, C.c_char_p]),
    "krk_cuda_nccl_comm_destroy": (_int, [_vp]),
    "krk_cuda_nccl_last_error": (C.c_char_p, []),
    "krk_cuda_moe_workspace_bytes": (_sz, [C.POINTER(ExpertBank), _int, _i64]),
    "krk_cuda_moe_ffn": (_int, [_vp, _vp, _vp, _vp, C.POINTER(ExpertBank), _int, _i64, _vp, _sz, _vp]),
    "krk_cuda_moe_ffn_routed": (_int, [_vp, _vp, _vp, _int, _vp, _vp, C.POINTER(ExpertBank), _int, _i64, _vp, _sz, _vp]),
    "krk_cuda_silu_mul": (_int, [_vp, _vp, _vp, _i64, _vp]),
    "krk_cuda_gather_rows": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "krk_cuda_scatter_axpy_rows": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "krk_cuda_sum_parts": (_int, [_vp, _vp, _int, _i64, _vp]),
    "krk_cuda_gemv_allgather": (_int, [C.POINTER(_vp), C.POINTER(_vp), _int, _int, _int, _int, _i64, _i64, _vp, _vp, _int, _i64,
                                       _i64, _i64, _vp]),
    "krk_cuda_wait_flags": (_int, [_vp, _int, _int, _vp]),
    "krk_cuda_embed": (_int, [_vp, _vp, _int, _i64, _i64, _vp, _i64, _vp]),
    "krk_cuda_logits_topk_workspace_bytes": (_sz, [_i64, _int]),
    "krk_cuda_logits_topk": (_int, [_vp, _i64, _int, _vp, C.c_float, C.c_float, C.c_float, _vp, _vp, _vp, _vp, _sz, _vp]),
    "krk_cuda_allgather_sum": (_int, [C.POINTER(_vp), C.POINTER(_vp), _int, _int, _i64, _vp, _vp, _i64, _vp]),
    "krk_cuda_peer_alloc": (_int, [C.POINTER(_vp), C.c_size_t, C.c_char_p]),
    "krk_cuda_peer_open": (_int, [C.POINTER(_vp), C.c_char_p]),
    "krk_cuda_peer_close": (_int, [_vp]),
    "krk_cuda_peer_free": (_int, [_vp]),
    "krk_cuda_device_status": (_int, []),
    "krk_cuda_launch_count": (_i64, []),
    "krk_cuda_family_count": (_i64, [_int]),
    "krk_cuda_probe_issue": (_int, [_int, _int, _int, _int, C.POINTER(C.c_double)]),
    "krk_cuda_backend_make": (_vp, [_int, C.c_char_p, _sz]),
    "krk_cuda_backend_free": (None, [_vp]),
    "krk_cuda_backend_describe": (C.c_char_p, [_vp]),
    "krk_cuda_backend_alloc": (_vp, [_vp, _sz]),
    "krk_cuda_backend_release": (None, [_vp, _vp]),
    "krk_cuda_backend_upload": (None, [_vp, _vp, _vp, _sz, _sz]),
    "krk_cuda_backend_download": (None, [_vp, _vp, _vp, _sz, _sz]),
    "krk_cuda_backend_download_f32": (None, [_vp, _vp, _vp, _i64]),
    "krk_cuda_backend_upload_i32": (None, [_vp, _vp, _vp, _i64]),
    "krk_cuda_backend_embed": (None, [_vp, _vp, _vp, _int, _i64, _i64, _vp, _i64]),
    "krk_cuda_backend_logits_topk": (None, [_vp, _vp, _i64, C.c_int32, _vp, C.c_float, C.c_float, C.c_float, _vp, _vp, _vp, _vp,
                                            C.c_int32, _vp]),
    "krk_cuda_backend_silu_mul": (None, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "krk_cuda_backend_gather_rows": (None, [_vp, _vp, _vp, _vp, _i64, _i64]),
    "krk_cuda_backend_scatter_axpy_rows": (None, [_vp, _vp, _vp, _vp, _vp, _i64, _i64]),
    "krk_cuda_backend_router_softmax": (None, [_vp, _vp, _vp, _i64, C.c_int32]),
    "krk_cuda_backend_router_topk": (None, [_vp, _vp, _i64, C.c_int32, C.c_int32, _vp, _vp, C.c_int32, C.c_float]),
    "krk_cuda_backend_moe_plan_build": (None, [_vp, _vp, _i64, C.c_int32, C.c_int32, _vp, _vp, _vp, _vp]),
    "krk_cuda_backend_device": (_int, [_vp]),
    "krk_gguf_open": (_vp, [C.c_char_p, C.c_char_p, _sz]),
    "krk_gguf_close": (None, [_vp]),
    "krk_gguf_version": (_int, [_vp]),
    "krk_gguf_tensor_count": (_i64, [_vp]),
    "krk_gguf_kv_count": (_i64, [_vp]),
    "krk_gguf_find_tensor": (_i64, [_vp, C.c_char_p]),
    "krk_gguf_tensor_info": (_int, [_vp, _i64, C.POINTER(GgufTensorInfo)]),
    "krk_gguf_get_i64": (_int, [_vp, C.c_char_p, C.POINTER(_i64)]),
    "krk_gguf_get_f64": (_int, [_vp, C.c_char_p, C.POINTER(C.c_double)]),
    "krk_gguf_get_str": (_i64, [_vp, C.c_char_p, C.c_char_p, _sz]),
    "krk_gguf_get_array_count": (_i64, [_vp, C.c_char_p, C.POINTER(_int)]),
    "krk_gguf_upload_tensor": (_vp, [_vp, _i64, _vp]),
    "krk_cuda_backend_fill0": (None, [_vp, _vp, _sz]),
    "krk_cuda_backend_sync": (None, [_vp]),
    "krk_cuda_backend_gemm_k_ok": (_int, [_vp, _int, _i64]),
    "krk_cuda_backend_gemm": (None, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64]),
    "krk_cuda_backend_gemm_accumulate": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64]),
    "krk_cuda_backend_gemm_group": (_int, [_vp, C.POINTER(_vp), _vp, C.POINTER(_vp), _int, C.POINTER(_i64),
                                           _i64, _int, _i64, _int, C.POINTER(_int)]),
    "krk_cuda_backend_gemm_group_ex": (_int, [_vp, C.POINTER(_vp), _vp, C.POINTER(_vp), _int, C.POINTER(_i64),
                                              _i64, _int, _i64, _int, C.POINTER(_int), C.POINTER(_int), C.POINTER(_vp)]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)   # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


def _check(rc: int, where: str) -> None:
    if rc != 0:
        raise KrkCudaError(rc, where)


def _stream_ptr(stream=None):
    """cudaStream_t of a torch stream (None = torch's current stream)."""
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


# ---- geometry ---------------------------------------------------------------------------

def row_bytes(wt: int, n_in: int) -> int:
    return lib.krk_cuda_row_bytes(wt, n_in)


def gemm_k_ok(wt: int, k: int) -> bool:
    return bool(lib.krk_cuda_gemm_k_ok(wt, k))


# ---- device-pointer entries ----------------------------------------------------------------

def dequant_rows(w, wt: int, n_rows: int, n_in: int, stream=None):
    import torch
    out = torch.empty((n_rows, n_in), dtype=torch.float32, device=w.device)
    _check(lib.krk_cuda_dequant_rows(_ptr(out), _ptr(w), wt, n_rows, n_in, _stream_ptr(stream)), "dequant_rows")
    return out


def gemv(x, w, wt: int, n_out: int, n_in: int, out=None, accumulate: bool = False, stream=None):
    """y[rows][n_out] (+)= x[rows][n_in] . W^T; x is f32 [rows, n_in] or [n_in]."""
    import torch
    rows = 1 if x.dim() == 1 else x.shape[0]
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an existing output")
        out = torch.empty((rows, n_out), dtype=torch.float32, device=x.device)
    _check(lib.krk_cuda_gemv(_ptr(out), _ptr(x), _ptr(w), wt, n_out, n_in, rows, int(accumulate),
                             _stream_ptr(stream)), "gemv")
    return out


def gemv_group(xs, ws, wts, n_outs, n_in: int, outs=None, fuse_silu_pair: bool = False, stream=None):
    """One launch for up to 16 single-row GEMVs. xs/ws/outs are lists of tensors."""
    import torch
    n = len(ws)
    if outs is None:
        outs = [torch.empty((n_outs[m],), dtype=torch.float32, device=ws[m].device) for m in range(n)]
    ya = (_vp * n)(*[t.data_ptr() for t in outs])
    xa = (_vp * n)(*[t.data_ptr() for t in xs])
    wa = (_vp * n)(*[t.data_ptr() for t in ws])
    ta = (_int * n)(*wts)
    na = (_i64 * n)(*n_outs)
    _check(lib.krk_cuda_gemv_group(ya, xa, wa, ta, na, n_in, n, int(fuse_silu_pair), _stream_ptr(stream)),
           "gemv_group")
    return outs


def gemm_workspace_bytes(x_dtype: int, n_out: int, n_in: int, rows: int) -> int:
    return lib.krk_cuda_gemm_workspace_bytes(x_dtype, n_out, n_in, rows)


def gemm(x, w, wt: int, n_out: int, n_in: int, out=None, workspace=None, stream=None):
    """Prefill GEMM: x is f16 or f32 [rows, n_in]; returns f32 [rows, n_out]."""
    import torch
    rows = x.shape[0]
    x_dtype = X_F16 if x.dtype == torch.float16 else X_F32
    need = gemm_workspace_bytes(x_dtype, n_out, n_in, rows)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty((rows, n_out), dtype=torch.float32, device=x.device)
    _check(lib.krk_cuda_gemm(_ptr(out), _ptr(x), x_dtype, _ptr(w), wt, n_out, n_in, rows, _ptr(workspace),
                             workspace.numel() if workspace is not None else 0, _stream_ptr(stream)), "gemm")
    return out


def gemm_f32_static(x, w, wt: int, n_out: int, n_in: int, out=None, stream=None):
    """krk_cuda_gemm_f32_static: f32 x [rows, n_in] -> f32 [rows, n_out], scratch inside the library."""
    import torch
    rows = x.shape[0]
    if out is None:
        out = torch.empty((rows, n_out), dtype=torch.float32, device=x.device)
    _check(lib.krk_cuda_gemm_f32_static(_ptr(out), _ptr(x), _ptr(w), wt, n_out, n_in, rows, _stream_ptr(stream)),
           "gemm_f32_static")
    return out


def gemm_f32_static_status() -> int:
    return lib.krk_cuda_gemm_f32_static_status()


def route(logits, k: int, stream=None):
    import torch
    n_tok, n_expert = logits.shape
    ids = torch.empty((n_tok, k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((n_tok, k), dtype=torch.float32, device=logits.device)
    _check(lib.krk_cuda_route(_ptr(ids), _ptr(wts), _ptr(logits), n_tok, n_expert, k, _stream_ptr(stream)), "route")
    return ids, wts


def router_softmax(logits, stream=None):
    import torch
    probs = torch.empty_like(logits)
    _check(lib.krk_cuda_router_softmax(_ptr(probs), _ptr(logits), logits.shape[0], logits.shape[1], _stream_ptr(stream)),
           "router_softmax")
    return probs


def router_topk(probs, k: int, normalize: bool = True, scale: float = 1.0, stream=None):
    import torch
    n_rows, n_expert = probs.shape
    ids = torch.empty((n_rows, k), dtype=torch.int32, device=probs.device)
    wts = torch.empty((n_rows, k), dtype=torch.float32, device=probs.device)
    _check(lib.krk_cuda_router_topk(_ptr(probs), n_rows, n_expert, k, _ptr(ids), _ptr(wts), int(normalize), scale,
                                    _stream_ptr(stream)), "router_topk")
    return ids, wts


def moe_plan_build(ids, wts, n_expert: int, stream=None):
    """Expert-major plan of a layer: (off int32 [n_expert + 1], rows int32 [n * k], wt f32 [n * k])."""
    import torch
    n_rows, k = ids.shape
    off = torch.empty(n_expert + 1, dtype=torch.int32, device=ids.device)
    rows = torch.full((n_rows * k,), -1, dtype=torch.int32, device=ids.device)
    wt = torch.zeros(n_rows * k, dtype=torch.float32, device=ids.device)
    _check(lib.krk_cuda_moe_plan_build(_ptr(ids), n_rows, k, n_expert, _ptr(off), _ptr(rows), _ptr(wt),
                                       _ptr(wts) if wts is not None else None, _stream_ptr(stream)), "moe_plan_build")
    return off, rows, wt


class NcclComm:
    """An NCCL communicator made through the library's own wrappers (krk_cuda_nccl_*), for the C-side
    all-gather krk_cuda_shard_allgather."""

    def __init__(self, n_ranks: int, rank: int, unique_id: bytes):
        self.h = _vp()
        _check(lib.krk_cuda_nccl_comm_init(C.byref(self.h), n_ranks, rank, unique_id), "nccl_comm_init")
        self.n_ranks, self.rank = n_ranks, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _check(lib.krk_cuda_nccl_unique_id(buf), "nccl_unique_id")
        return buf.raw

    def allgather(self, full, slice_, stream=None):
        nbytes = slice_.numel() * slice_.element_size()
        _check(lib.krk_cuda_shard_allgather(_ptr(full), _ptr(slice_), nbytes, self.h, _stream_ptr(stream)), "shard_allgather")
        return full

    def close(self):
        if self.h:
            lib.krk_cuda_nccl_comm_destroy(self.h)
            self.h = _vp()


def make_bank(gate, up, down, wt_gate_up: int, wt_down: int, n_local: int, expert_base: int, n_embd: int,
              n_ff: int) -> ExpertBank:
    bank = ExpertBank(gate.data_ptr() if gate is not None else 0, up.data_ptr() if up is not None else 0,
                      down.data_ptr() if down is not None else 0, wt_gate_up, wt_down, n_local, expert_base,
                      n_embd, n_ff)
    bank._keep = (gate, up, down)   # the struct holds raw pointers: keep the tensors alive with it
    return bank


def moe_ffn(x, ids, wts, bank: ExpertBank, out=None, workspace=None, stream=None):
    import torch
    n_tok, k = ids.shape
    need = lib.krk_cuda_moe_workspace_bytes(C.byref(bank), k, n_tok)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty((n_tok, bank.n_embd), dtype=torch.float32, device=x.device)
    _check(lib.krk_cuda_moe_ffn(_ptr(out), _ptr(x), _ptr(ids), _ptr(wts), C.byref(bank), k, n_tok, _ptr(workspace),
                                workspace.numel(), _stream_ptr(stream)), "moe_ffn")
    return out


def moe_ffn_routed(x, logits, k: int, bank: ExpertBank, out=None, workspace=None, stream=None):
    """Routing + routed-expert FFN in one call. Returns (y, ids, wts); ids / wts are what route() gives."""
    import torch
    n_tok, n_expert = logits.shape
    ids = torch.empty((n_tok, k), dtype=torch.int32, device=x.device)
    wts = torch.empty((n_tok, k), dtype=torch.float32, device=x.device)
    need = lib.krk_cuda_moe_workspace_bytes(C.byref(bank), k, n_tok)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty((n_tok, bank.n_embd), dtype=torch.float32, device=x.device)
    _check(lib.krk_cuda_moe_ffn_routed(_ptr(out), _ptr(x), _ptr(logits), n_expert, _ptr(ids), _ptr(wts), C.byref(bank), k,
                                       n_tok, _ptr(workspace), workspace.numel(), _stream_ptr(stream)), "moe_ffn_routed")
    return out, ids, wts


def silu_mul(gate, up, out=None, stream=None):
    import torch
    if out is None:
        out = torch.empty_like(gate)
    _check(lib.krk_cuda_silu_mul(_ptr(out), _ptr(gate), _ptr(up), gate.numel(), _stream_ptr(stream)), "silu_mul")
    return out


def gather_rows(dst, src, rows, stream=None):
    """dst[i] = src[rows[i]]; dst [n_rows][n] f32, rows device i32."""
    _check(lib.krk_cuda_gather_rows(_ptr(dst), _ptr(src), _ptr(rows), dst.shape[0], dst.shape[1],
                                    _stream_ptr(stream)), "gather_rows")
    return dst


def scatter_axpy_rows(dst, src, rows, alpha, stream=None):
    _check(lib.krk_cuda_scatter_axpy_rows(_ptr(dst), _ptr(src), _ptr(rows), _ptr(alpha), src.shape[0],
                                          src.shape[1], _stream_ptr(stream)), "scatter_axpy_rows")
    return dst


def sum_parts(parts, out=None, stream=None):
    import torch
    n_parts = parts.shape[0]
    n = parts[0].numel()
    if out is None:
        out = torch.empty_like(parts[0])
    _check(lib.krk_cuda_sum_parts(_ptr(out), _ptr(parts), n_parts, n, _stream_ptr(stream)), "sum_parts")
    return out


def gemv_allgather(y_peer_ptrs, flag_peer_ptrs, my_rank: int, epoch: int, slice_offset: int, n_out_total: int, x, w,
                   wt: int, n_out_local: int, n_in: int, wait_in_kernel: bool = True, stream=None):
    """Fused row-sharded GEMV + all-gather: y_peer_ptrs / flag_peer_ptrs are device addresses (ints) of every
    GPU's full output buffer and flag array as mapped into this process."""
    n = len(y_peer_ptrs)
    rows = 1 if x.dim() == 1 else x.shape[0]
    _check(lib.krk_cuda_gemv_allgather((_vp * n)(*y_peer_ptrs), (_vp * n)(*flag_peer_ptrs), n, my_rank, epoch, int(wait_in_kernel), slice_offset,
                                       n_out_total, _ptr(x), _ptr(w), wt, n_out_local, n_in, rows, _stream_ptr(stream)),
           "gemv_allgather")


def wait_flags(flags, n_peers: int, epoch: int, stream=None):
    _check(lib.krk_cuda_wait_flags(_ptr(flags), n_peers, epoch, _stream_ptr(stream)), "wait_flags")


def embed(table, wt: int, n_vocab: int, n_embd: int, tokens, out=None, stream=None):
    """Rows of a quantized embedding table by token id (device int32 tensor) as f32; bad ids give zero rows."""
    import torch
    n_tok = tokens.numel()
    if out is None:
        out = torch.empty((n_tok, n_embd), dtype=torch.float32, device=table.device)
    _check(lib.krk_cuda_embed(_ptr(out), _ptr(table), wt, n_vocab, n_embd, _ptr(tokens), n_tok, _stream_ptr(stream)), "embed")
    return out


def logits_topk(logits, k: int, pen_mask=None, rep_pen: float = 1.0, softcap: float = 0.0, temp: float = 1.0,
                want_mass: bool = True, workspace=None, stream=None):
    """Device top-k of one f32 logits row: (ids int32 [k], vals f32 [k], mass f32 [1] or None)."""
    import torch
    n = logits.numel()
    ids = torch.empty(k, dtype=torch.int32, device=logits.device)
    vals = torch.empty(k, dtype=torch.float32, device=logits.device)
    mass = torch.empty(1, dtype=torch.float32, device=logits.device) if want_mass else None
    need = lib.krk_cuda_logits_topk_workspace_bytes(n, k)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=logits.device)
    _check(lib.krk_cuda_logits_topk(_ptr(logits), n, k, _ptr(pen_mask) if pen_mask is not None else None, rep_pen, softcap,
                                    temp, _ptr(ids), _ptr(vals), _ptr(mass) if mass is not None else None, _ptr(workspace),
                                    workspace.numel(), _stream_ptr(stream)), "logits_topk")
    return ids, vals, mass


def allgather_sum(gather_peer_ptrs, flag_peer_ptrs, my_rank: int, slot_stride: int, part, out, stream=None):
    """Exchange step of an expert-sharded FFN: all-gather of `part` over peer stores + rank-ordered sum."""
    n = len(gather_peer_ptrs)
    _check(lib.krk_cuda_allgather_sum((_vp * n)(*gather_peer_ptrs), (_vp * n)(*flag_peer_ptrs), n, my_rank, slot_stride,
                                      _ptr(part), _ptr(out), part.numel(), _stream_ptr(stream)), "allgather_sum")
    return out


class PeerBuffer:
    """Device memory that other processes of the box can map (krk_cuda_peer_alloc / _open). ``tensor``
    views it as a torch tensor on ``device`` (the accessor's device for a mapped buffer: the address is
    only ever handed to this library's kernels, which store through NVLink)."""

    def __init__(self, ptr: int, nbytes: int, handle: bytes, owned: bool):
        self.ptr, self.nbytes, self.handle, self.owned = ptr, nbytes, handle, owned

    @classmethod
    def alloc(cls, nbytes: int) -> "PeerBuffer":
        ptr, handle = _vp(), C.create_string_buffer(64)
        _check(lib.krk_cuda_peer_alloc(C.byref(ptr), nbytes, handle), "peer_alloc")
        return cls(ptr.value, nbytes, handle.raw, True)

    @classmethod
    def open(cls, handle: bytes, nbytes: int) -> "PeerBuffer":
        ptr = _vp()
        _check(lib.krk_cuda_peer_open(C.byref(ptr), handle), "peer_open")
        return cls(ptr.value, nbytes, handle, False)

    def tensor(self, shape, dtype):
        """The buffer as a tensor of the current device (own buffers only)."""
        import torch
        if not self.owned:
            raise ValueError("a mapped peer buffer is only addressed by kernels of this library")
        itemsize = torch.empty(0, dtype=dtype).element_size()
        typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]
        n = 1
        for d in shape:
            n *= int(d)
        if n * itemsize > self.nbytes:
            raise ValueError("view larger than the buffer")

        class _View:
            __cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (self.ptr, False), "version": 2}
        t = torch.as_tensor(_View(), device=torch.device("cuda", torch.cuda.current_device()))
        t._krk_owner = self
        return t

    def release(self):
        if self.ptr:
            (lib.krk_cuda_peer_free if self.owned else lib.krk_cuda_peer_close)(self.ptr)
            self.ptr = 0


def device_status() -> int:
    return lib.krk_cuda_device_status()


def launch_count() -> int:
    return lib.krk_cuda_launch_count()


FAMILY_GEMV_STREAM, FAMILY_GEMV_GENERIC, FAMILY_GEMM_TC = 1, 2, 3


def family_count(family: int) -> int:
    return lib.krk_cuda_family_count(family)


PROBE_KINDS = ("mma.sync.m16n8k32.s8", "mma.sync.m16n8k16.s8", "mma.sync.m16n8k16.f16", "mma.sync.m16n8k16.bf16",
               "mma.sync.m16n8k32.e4m3", "dp4a.s32", "mad.lo.s32", "fma.rn.f16x2", "lop3.b32", "fma.rn.f32",
               "mma.sync.m16n8k8.f16")


def probe_issue(kind: int, warps: int, iters: int = 4096, chained: bool = False) -> float:
    """Cycles per instruction of one kind on one SM sub-partition (krk_cuda_probe_issue)."""
    out = C.c_double(0.0)
    _check(lib.krk_cuda_probe_issue(kind, warps, iters, int(chained), C.byref(out)), "probe_issue")
    return out.value


# ---- host-buffer plumbing: the CudaBackend object ---------------------------------------------

class Backend:
    """The C++ CudaBackend (include/krk_cuda_backend.hpp) driven through its C shim.

    Mirrors the members of krk::Backend this path needs; host arrays are numpy arrays or
    pinned torch tensors, device memory comes from alloc().
    """

    def __init__(self, device_index: int = 0):
        err = C.create_string_buffer(256)
        self.h = lib.krk_cuda_backend_make(device_index, err, 256)
        if not self.h:
            raise RuntimeError(f"make_cuda_backend({device_index}) failed: {err.value.decode()}")

    def close(self):
        if self.h:
            lib.krk_cuda_backend_free(self.h)
            self.h = None

    def describe(self) -> str:
        return lib.krk_cuda_backend_describe(self.h).decode()

    def alloc(self, nbytes: int) -> int:
        p = lib.krk_cuda_backend_alloc(self.h, nbytes)
        if not p:
            raise MemoryError(f"backend alloc of {nbytes} bytes failed")
        return p

    def release(self, p: int) -> None:
        lib.krk_cuda_backend_release(self.h, p)

    def upload(self, dst: int, host_ptr: int, nbytes: int, off: int = 0) -> None:
        lib.krk_cuda_backend_upload(self.h, dst, host_ptr, nbytes, off)

    def download(self, host_ptr: int, src: int, nbytes: int, off: int = 0) -> None:
        lib.krk_cuda_backend_download(self.h, host_ptr, src, nbytes, off)

    def router_softmax(self, probs: int, logits: int, n_rows: int, n_expert: int) -> None:
        lib.krk_cuda_backend_router_softmax(self.h, probs, logits, n_rows, n_expert)

    def router_topk(self, probs: int, n_rows: int, n_expert: int, k: int, ids: int, wts: int, normalize: bool = True,
                    scale: float = 1.0) -> None:
        lib.krk_cuda_backend_router_topk(self.h, probs, n_rows, n_expert, k, ids, wts, int(normalize), scale)

    def moe_plan_build(self, ids: int, n_rows: int, k: int, n_expert: int, off: int, rows: int, wt: int, wts: int) -> None:
        lib.krk_cuda_backend_moe_plan_build(self.h, ids, n_rows, k, n_expert, off, rows, wt, wts)

    def fill0(self, p: int, nbytes: int) -> None:
        lib.krk_cuda_backend_fill0(self.h, p, nbytes)

    def sync(self) -> None:
        lib.krk_cuda_backend_sync(self.h)

    def gemm_k_ok(self, wt: int, k: int) -> bool:
        return bool(lib.krk_cuda_backend_gemm_k_ok(self.h, wt, k))

    def gemm(self, out: int, x: int, w: int, wt: int, n_out: int, n_in: int, rows: int) -> None:
        lib.krk_cuda_backend_gemm(self.h, out, x, w, wt, n_out, n_in, rows)

    def gemm_accumulate(self, dst: int, x: int, w: int, wt: int, n_out: int, n_in: int, rows: int) -> bool:
        return bool(lib.krk_cuda_backend_gemm_accumulate(self.h, dst, x, w, wt, n_out, n_in, rows))

    def gemm_group(self, outs, x: int, ws, wt: int, n_outs, n_in: int, rows: int = 1, silu: bool = False,
                   wts=None, xs=None):
        """Backend::gemm_group; wts / xs are its optional per-matrix weight types and activations."""
        n = len(ws)
        fused = _int(0)
        if wts is None and xs is None:
            ran = lib.krk_cuda_backend_gemm_group(self.h, (_vp * n)(*outs), x, (_vp * n)(*ws), wt, (_i64 * n)(*n_outs),
                                                  n_in, n, rows, int(silu), C.byref(fused))
        else:
            ran = lib.krk_cuda_backend_gemm_group_ex(self.h, (_vp * n)(*outs), x, (_vp * n)(*ws), wt, (_i64 * n)(*n_outs),
                                                     n_in, n, rows, int(silu), C.byref(fused),
                                                     (_int * n)(*wts) if wts is not None else None,
                                                     (_vp * n)(*xs) if xs is not None else None)
        return bool(ran), bool(fused.value)


class Gguf:
    """A GGUF file through the library's reader (krk_gguf_*): tensors as views of the mapped file."""

    def __init__(self, path: str):
        err = C.create_string_buffer(256)
        self.h = lib.krk_gguf_open(path.encode(), err, 256)
        if not self.h:
            raise ValueError(f"{path}: {err.value.decode()}")

    def close(self):
        if self.h:
            lib.krk_gguf_close(self.h)
            self.h = None

    @property
    def version(self) -> int:
        return lib.krk_gguf_version(self.h)

    def __len__(self) -> int:
        return lib.krk_gguf_tensor_count(self.h)

    def kv_count(self) -> int:
        return lib.krk_gguf_kv_count(self.h)

    def info(self, index: int) -> GgufTensorInfo:
        out = GgufTensorInfo()
        _check(lib.krk_gguf_tensor_info(self.h, index, C.byref(out)), "gguf_tensor_info")
        return out

    def find(self, name: str) -> int:
        return lib.krk_gguf_find_tensor(self.h, name.encode())

    def tensor_bytes(self, index: int):
        """uint8 numpy copy of the tensor's bytes."""
        import numpy as np
        t = self.info(index)
        if not t.n_bytes:
            raise ValueError("a tensor of a type this library does not size")
        return np.ctypeslib.as_array(C.cast(t.host_data, C.POINTER(C.c_uint8)), shape=(t.n_bytes,)).copy()

    def get_int(self, key: str):
        out = _i64(0)
        return out.value if lib.krk_gguf_get_i64(self.h, key.encode(), C.byref(out)) == 0 else None

    def get_float(self, key: str):
        out = C.c_double(0.0)
        return out.value if lib.krk_gguf_get_f64(self.h, key.encode(), C.byref(out)) == 0 else None

    def get_str(self, key: str):
        n = lib.krk_gguf_get_str(self.h, key.encode(), None, 0)
        if n < 0:
            return None
        buf = C.create_string_buffer(n + 1)
        lib.krk_gguf_get_str(self.h, key.encode(), buf, n + 1)
        return buf.value.decode(errors="replace")

    def array_count(self, key: str):
        et = _int(0)
        n = lib.krk_gguf_get_array_count(self.h, key.encode(), C.byref(et))
        return (n, et.value) if n >= 0 else None

    def upload(self, index: int, backend: "Backend") -> int:
        p = lib.krk_gguf_upload_tensor(self.h, index, backend.h)
        if not p:
            raise MemoryError("gguf upload failed (unsized type or allocation)")
        return p
