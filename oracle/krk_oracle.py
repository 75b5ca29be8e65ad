"""ctypes face of the CPU checker (libkrk_oracle.so) and, when built, of the compiled
reference (oracle/_ref/libkrk_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline / reference arms. The product package never imports this module.
Parity status: pinned (see krk_oracle.h).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libkrk_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libkrk_ref.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build(with_ref: bool = True) -> None:
    """Compile the restatement and, if the reference tree is mounted, oracle/_ref."""
    targets = ["all"] + (["ref"] if with_ref else [])
    env = dict(os.environ)
    if "KRK_REF" not in env:
        # a Kraken tree checked out beside this repository as `reference`; elsewhere set KRK_REF (without
        # either, `make ref` keeps whatever prebuilt oracle/_ref travelled with the tree)
        cand = os.path.join(os.path.dirname(os.path.dirname(_HERE.rstrip(os.sep))), "reference")
        if os.path.isdir(os.path.join(cand, "src")):
            env["KRK_REF"] = cand
    subprocess.run(["make", "-C", _HERE] + targets, check=True, stdout=subprocess.DEVNULL, env=env)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


class Oracle:
    """The C restatement of the reference's scalar f32 path."""

    kind = "port"

    def __init__(self):
        if not os.path.exists(_ORACLE_SO):
            build(with_ref=False)
        L = C.CDLL(_ORACLE_SO)
        L.krk_oracle_block_size.restype = C.c_int
        L.krk_oracle_block_bytes.restype = C.c_int
        L.krk_oracle_row_bytes.restype = C.c_size_t
        L.krk_oracle_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.krk_oracle_fp16_to_fp32.restype = C.c_float
        L.krk_oracle_fp16_to_fp32.argtypes = [C.c_uint16]
        L.krk_oracle_dequant_rows.argtypes = [_f32p, _u8p, C.c_int, C.c_int64, C.c_int64]
        L.krk_oracle_gemm.argtypes = [_f32p, _f32p, _u8p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int]
        L.krk_oracle_route.argtypes = [_i32p, _f32p, _f32p, C.c_int64, C.c_int, C.c_int]
        L.krk_oracle_silu_mul.argtypes = [_f32p, _f32p, _f32p, C.c_int64]
        L.krk_oracle_silu_mul.restype = None
        L.krk_oracle_scatter_axpy_rows.argtypes = [_f32p, _f32p, _i32p, _f32p, C.c_int64, C.c_int64]
        L.krk_oracle_scatter_axpy_rows.restype = None
        L.krk_oracle_embed.argtypes = [_f32p, _u8p, C.c_int, C.c_int64, C.c_int64, _i32p, C.c_int64]
        L.krk_oracle_logits_topk.argtypes = [_f32p, C.c_int64, C.c_int, C.c_void_p, C.c_float, C.c_float, C.c_float, _i32p,
                                             _f32p, _f32p]
        L.krk_oracle_moe_ffn.argtypes = [_f32p, _f32p, _i32p, _f32p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64,
                                         C.c_int64, C.c_int]
        self.L = L

    def block_size(self, wt):
        return self.L.krk_oracle_block_size(wt)

    def block_bytes(self, wt):
        return self.L.krk_oracle_block_bytes(wt)

    def row_bytes(self, wt, n_in):
        return self.L.krk_oracle_row_bytes(wt, n_in)

    def fp16_to_fp32(self, h):
        return self.L.krk_oracle_fp16_to_fp32(int(h))

    def dequant_rows(self, w, wt, n_rows, n_in):
        w = _c(w, np.uint8).reshape(-1)
        out = np.empty((n_rows, n_in), dtype=np.float32)
        rc = self.L.krk_oracle_dequant_rows(out.reshape(-1), w, wt, n_rows, n_in)
        if rc != 0:
            raise ValueError(f"dequant_rows refused wt={wt} n_in={n_in}")
        return out

    def gemm(self, x, w, wt, n_out, n_in, rows=1, threads=1):
        x = _c(x, np.float32).reshape(-1)
        w = _c(w, np.uint8).reshape(-1)
        out = np.empty((rows, n_out), dtype=np.float32)
        rc = self.L.krk_oracle_gemm(out.reshape(-1), x, w, wt, n_out, n_in, rows, threads)
        if rc != 0:
            raise ValueError(f"gemm refused wt={wt} n_out={n_out} n_in={n_in} rows={rows}")
        return out

    def route(self, logits, k):
        logits = _c(logits, np.float32)
        n_tok, n_expert = logits.shape
        ids = np.empty((n_tok, k), dtype=np.int32)
        wts = np.empty((n_tok, k), dtype=np.float32)
        rc = self.L.krk_oracle_route(ids.reshape(-1), wts.reshape(-1), logits.reshape(-1), n_tok, n_expert, k)
        if rc != 0:
            raise ValueError("route refused its arguments")
        return ids, wts

    def embed(self, table, wt, n_vocab, n_embd, tokens):
        table, tokens = _c(table, np.uint8), _c(tokens, np.int32)
        out = np.empty((tokens.size, n_embd), dtype=np.float32)
        fn = getattr(self.L, "krk_oracle_embed", None) or self.L.krk_ref_embed
        fn(out, table.reshape(-1), wt, n_vocab, n_embd, tokens.reshape(-1), tokens.size)
        return out

    def logits_topk(self, logits, k, pen_mask=None, rep_pen=1.0, softcap=0.0, temp=1.0):
        logits = _c(logits, np.float32).reshape(-1)
        ids = np.empty(k, dtype=np.int32)
        vals = np.empty(k, dtype=np.float32)
        mass = np.empty(1, dtype=np.float32)
        pm = None if pen_mask is None else _c(pen_mask, np.uint32)
        fn = getattr(self.L, "krk_oracle_logits_topk", None) or self.L.krk_ref_logits_topk
        fn(logits, logits.size, k, None if pm is None else pm.ctypes.data_as(C.c_void_p), rep_pen, softcap, temp, ids, vals, mass)
        return ids, vals, float(mass[0])

    def silu_mul(self, gate, up):
        gate = _c(gate, np.float32)
        up = _c(up, np.float32)
        out = np.empty_like(gate)
        self.L.krk_oracle_silu_mul(out.reshape(-1), gate.reshape(-1), up.reshape(-1), gate.size)
        return out

    @staticmethod
    def gather_rows(src, rows):
        """dst[i * n + j] = src[rows[i] * n + j] (include/krk/backend.hpp:1443-1452): a move of f32 rows, no
        arithmetic."""
        return np.ascontiguousarray(_c(src, np.float32)[np.asarray(rows, np.int64)])

    def scatter_axpy_rows(self, dst, src, rows, alpha):
        src = _c(src, np.float32)
        self.L.krk_oracle_scatter_axpy_rows(dst.reshape(-1), src.reshape(-1), _c(rows, np.int32),
                                            _c(alpha, np.float32), src.shape[0], src.shape[1])
        return dst

    def moe_ffn(self, x, ids, wts, gate, up, down, wt_gate_up, wt_down, n_embd, n_ff, threads=1):
        """gate/up/down: lists of uint8 arrays or None (expert not held by this shard)."""
        x = _c(x, np.float32)
        n_tok = x.shape[0]
        n_expert = len(gate)
        k = ids.shape[1]
        keep = []

        def ptrs(mats):
            arr = (C.c_void_p * n_expert)()
            for e, m in enumerate(mats):
                if m is None:
                    arr[e] = None
                else:
                    m = _c(m, np.uint8)
                    keep.append(m)
                    arr[e] = m.ctypes.data
            return arr

        y = np.empty((n_tok, n_embd), dtype=np.float32)
        rc = self.L.krk_oracle_moe_ffn(y.reshape(-1), x.reshape(-1), _c(ids, np.int32).reshape(-1),
                                       _c(wts, np.float32).reshape(-1), ptrs(gate), ptrs(up), ptrs(down),
                                       wt_gate_up, wt_down, n_expert, k, n_tok, n_embd, n_ff, threads)
        if rc != 0:
            raise ValueError("moe_ffn refused its arguments")
        return y


class Reference:
    """The reference's own compiled CPU path behind oracle/ref_shim.cpp."""

    kind = "reference"

    def __init__(self, threads: int | None = None):
        if not os.path.exists(_REF_SO):
            raise FileNotFoundError(_REF_SO)
        if threads is not None:
            # read once, when the reference creates its pool (src/par_pool.hpp:367-368)
            os.environ["KRK_THREADS"] = str(int(threads))
        L = C.CDLL(_REF_SO)
        L.krk_ref_fp16_to_fp32.restype = C.c_float
        L.krk_ref_fp16_to_fp32.argtypes = [C.c_uint16]
        L.krk_ref_fp32_to_fp16.restype = C.c_uint16
        L.krk_ref_fp32_to_fp16.argtypes = [C.c_float]
        L.krk_ref_row_bytes.restype = C.c_size_t
        L.krk_ref_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.krk_ref_dequant_rows.argtypes = [_f32p, _u8p, C.c_int, C.c_int64, C.c_int64]
        L.krk_ref_vec_dot.restype = C.c_float
        L.krk_ref_vec_dot.argtypes = [C.c_int, _u8p, _f32p, C.c_int64, C.c_int]
        L.krk_ref_gemm.argtypes = [_f32p, _f32p, _u8p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int]
        L.krk_ref_silu_mul.argtypes = [_f32p, _f32p, _f32p, C.c_int64]
        L.krk_ref_silu_mul.restype = None
        L.krk_ref_scatter_axpy_rows.argtypes = [_f32p, _f32p, _i32p, _f32p, C.c_int64, C.c_int64]
        L.krk_ref_scatter_axpy_rows.restype = None
        L.krk_ref_embed.argtypes = [_f32p, _u8p, C.c_int, C.c_int64, C.c_int64, _i32p, C.c_int64]
        L.krk_ref_embed.restype = None
        L.krk_ref_logits_topk.argtypes = [_f32p, C.c_int64, C.c_int, C.c_void_p, C.c_float, C.c_float, C.c_float, _i32p, _f32p,
                                          _f32p]
        L.krk_ref_logits_topk.restype = None
        self.L = L

    @staticmethod
    def available() -> bool:
        return os.path.exists(_REF_SO)

    def block_size(self, wt):
        return self.L.krk_ref_block_size(wt)

    def block_bytes(self, wt):
        return self.L.krk_ref_block_bytes(wt)

    def row_bytes(self, wt, n_in):
        return self.L.krk_ref_row_bytes(wt, n_in)

    def fp16_to_fp32(self, h):
        return self.L.krk_ref_fp16_to_fp32(int(h))

    def fp32_to_fp16(self, f):
        return self.L.krk_ref_fp32_to_fp16(float(f))

    def default_tiers(self):
        return self.L.krk_ref_default_tiers()

    def dequant_rows(self, w, wt, n_rows, n_in):
        w = _c(w, np.uint8).reshape(-1)
        out = np.empty((n_rows, n_in), dtype=np.float32)
        self.L.krk_ref_dequant_rows(out.reshape(-1), w, wt, n_rows, n_in)
        return out

    def vec_dot(self, wt, row, x, tier=0):
        x = _c(x, np.float32).reshape(-1)
        return self.L.krk_ref_vec_dot(wt, _c(row, np.uint8).reshape(-1), x, x.size, tier)

    def gemm(self, x, w, wt, n_out, n_in, rows=1, tier=0, threads=None):
        x = _c(x, np.float32).reshape(-1)
        w = _c(w, np.uint8).reshape(-1)
        out = np.empty((rows, n_out), dtype=np.float32)
        self.L.krk_ref_gemm(out.reshape(-1), x, w, wt, n_out, n_in, rows, tier)
        return out

    def embed(self, table, wt, n_vocab, n_embd, tokens):
        table, tokens = _c(table, np.uint8), _c(tokens, np.int32)
        out = np.empty((tokens.size, n_embd), dtype=np.float32)
        fn = getattr(self.L, "krk_oracle_embed", None) or self.L.krk_ref_embed
        fn(out, table.reshape(-1), wt, n_vocab, n_embd, tokens.reshape(-1), tokens.size)
        return out

    def logits_topk(self, logits, k, pen_mask=None, rep_pen=1.0, softcap=0.0, temp=1.0):
        logits = _c(logits, np.float32).reshape(-1)
        ids = np.empty(k, dtype=np.int32)
        vals = np.empty(k, dtype=np.float32)
        mass = np.empty(1, dtype=np.float32)
        pm = None if pen_mask is None else _c(pen_mask, np.uint32)
        fn = getattr(self.L, "krk_oracle_logits_topk", None) or self.L.krk_ref_logits_topk
        fn(logits, logits.size, k, None if pm is None else pm.ctypes.data_as(C.c_void_p), rep_pen, softcap, temp, ids, vals, mass)
        return ids, vals, float(mass[0])

    def silu_mul(self, gate, up):
        gate = _c(gate, np.float32)
        up = _c(up, np.float32)
        out = np.empty_like(gate)
        self.L.krk_ref_silu_mul(out.reshape(-1), gate.reshape(-1), up.reshape(-1), gate.size)
        return out

    def scatter_axpy_rows(self, dst, src, rows, alpha):
        src = _c(src, np.float32)
        self.L.krk_ref_scatter_axpy_rows(dst.reshape(-1), src.reshape(-1), _c(rows, np.int32),
                                         _c(alpha, np.float32), src.shape[0], src.shape[1])
        return dst
