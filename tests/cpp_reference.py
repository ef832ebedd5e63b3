"""The plain C++ restatements of the device operations (chibillm_b200/csrc/reference_ops.cc)
behind the call signatures of ``chibillm_b200.kernels.ops.CudaKernels``.

Arguments may live on any device and have any of the engine's types: they are
brought to the host as 32-bit floats (32-bit integers for index arrays), the
C++ loop runs, and the result is rounded into ``out`` where it lives.  For tests
only; it is slow by design.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from chibillm_b200.csrc import build

_F = ctypes.POINTER(ctypes.c_float)
_I = ctypes.POINTER(ctypes.c_int)
_LL = ctypes.c_longlong
_i = ctypes.c_int
_f = ctypes.c_float

_SIGNATURES = {
    "chibi_ref_embed": (_i, [_I, _F, _F, _LL, _i, _i]),
    "chibi_ref_rmsnorm": (None, [_F, _F, _F, _LL, _i, _f, _f]),
    "chibi_ref_linear": (None, [_F, _F, _F, _F, _LL, _i, _i]),
    "chibi_ref_swiglu": (None, [_F, _F, _LL, _i]),
    "chibi_ref_gather_rows": (None, [_F, _I, _F, _i, _i]),
    "chibi_ref_qk_norm_rope_append": (_i, [_F, _LL, _F, _F, _F, _F, _F, _F, _i, _f, _f, _I, _I, _I, _i,
                                           _i, _i, _i, _i, _i]),
    "chibi_ref_attention": (_i, [_F, _F, _F, _F, _I, _i, _I, _I, _LL, _i, _i, _i, _i, _i, _f, _i]),
    "chibi_ref_sample": (None, [_F, _LL, _i, _i, _F, _F, _I]),
}


def _host_f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().to("cpu", torch.float32).contiguous()


def _host_i32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().to("cpu", torch.int32).contiguous()


def _fp(t: Optional[torch.Tensor]):
    return ctypes.cast(0 if t is None else t.data_ptr(), _F)


def _ip(t: Optional[torch.Tensor]):
    return ctypes.cast(0 if t is None else t.data_ptr(), _I)


class CppReferenceKernels:
    name = "cpp-reference"

    def __init__(self):
        self.lib = ctypes.CDLL(build.reference_library(verbose=False))
        for fn, (restype, argtypes) in _SIGNATURES.items():
            getattr(self.lib, fn).restype = restype
            getattr(self.lib, fn).argtypes = argtypes

    def embed(self, tokens, table, out):
        tok, tab = _host_i32(tokens), _host_f32(table)
        res = torch.zeros(out.shape, dtype=torch.float32)
        bad = self.lib.chibi_ref_embed(_ip(tok), _fp(tab), _fp(res), tok.numel(), tab.shape[1], tab.shape[0])
        assert bad == 0, f"{bad} token ids outside the table"
        out.copy_(res.to(out.dtype))

    def rmsnorm(self, x, weight, eps, offset, out):
        xf, wf = _host_f32(x), _host_f32(weight)
        n = xf.shape[-1]
        res = torch.empty_like(xf)
        self.lib.chibi_ref_rmsnorm(_fp(xf), _fp(wf), _fp(res), xf.numel() // n, n, eps, offset)
        out.copy_(res.reshape(out.shape).to(out.dtype))

    def linear(self, x, w, out, residual=None, defer=False):
        xf, wf, rf = _host_f32(x), _host_f32(w), _host_f32(residual)
        M, K = xf.shape
        N = wf.shape[0]
        res = torch.empty(M, N, dtype=torch.float32)
        self.lib.chibi_ref_linear(_fp(xf), _fp(wf), _fp(rf), _fp(res), M, N, K)
        out.copy_(res.to(out.dtype))

    def swiglu(self, gate_up, out):
        gf = _host_f32(gate_up)
        res = torch.empty(out.shape, dtype=torch.float32)
        self.lib.chibi_ref_swiglu(_fp(gf), _fp(res), gf.shape[0], out.shape[1])
        out.copy_(res.to(out.dtype))

    def gather_rows(self, x, rows, out):
        xf, r = _host_f32(x), _host_i32(rows)
        res = torch.empty(out.shape, dtype=torch.float32)
        self.lib.chibi_ref_gather_rows(_fp(xf), _ip(r), _fp(res), r.numel(), xf.shape[1])
        out.copy_(res.to(out.dtype))

    def qk_norm_rope_append(self, qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq,
                            rotary_dim, eps, norm_offset, positions, seq_of_token, block_table,
                            nq, nkv, d, page_size, seq_rows=None):
        assert seq_rows is None
        T = qkv.shape[0]
        qf = _host_f32(qkv)
        qo = torch.zeros(T, nq * d, dtype=torch.float32)
        kc, vc = _host_f32(k_cache), _host_f32(v_cache)
        bt = _host_i32(block_table)
        # every host copy keeps a name until the call returns: a temporary would be freed under the pointer
        qw, kw, freq = _host_f32(q_norm_w), _host_f32(k_norm_w), _host_f32(inv_freq)
        pos, seq = _host_i32(positions), _host_i32(seq_of_token)
        bad = self.lib.chibi_ref_qk_norm_rope_append(
            _fp(qf), T, _fp(qo), _fp(kc), _fp(vc), _fp(qw), _fp(kw), _fp(freq), rotary_dim, eps, norm_offset,
            _ip(pos), _ip(seq), _ip(bt), 0 if bt is None else bt.shape[1], nq, nkv, d, page_size,
            0 if kc is None else kc.shape[0])
        assert bad == 0, f"{bad} tokens without a page"
        q_out.copy_(qo.to(q_out.dtype))
        if k_cache is not None:
            k_cache.copy_(kc.to(k_cache.dtype))
            v_cache.copy_(vc.to(v_cache.dtype))

    def attention(self, q, k_cache, v_cache, out, block_table, q_start, ctx_len, seq_of_token,
                  positions, nq, nkv, d, page_size, scale, window, max_q_len, max_ctx_len, min_q_len=0,
                  seq_rows=None):
        assert seq_rows is None
        T = q.shape[0]
        qf, kc, vc = _host_f32(q), _host_f32(k_cache), _host_f32(v_cache)
        bt = _host_i32(block_table)
        res = torch.zeros(T, nq * d, dtype=torch.float32)
        pos, seq = _host_i32(positions), _host_i32(seq_of_token)
        bad = self.lib.chibi_ref_attention(_fp(qf), _fp(kc), _fp(vc), _fp(res), _ip(bt), bt.shape[1], _ip(pos),
                                           _ip(seq), T, nq, nkv, d, page_size, kc.shape[0], scale, int(window or 0))
        assert bad == 0, f"{bad} rows read outside the pool"
        out.copy_(res.to(out.dtype))

    def sample(self, logits, temperature, uniform, out):
        lf = _host_f32(logits)
        res = torch.empty(lf.shape[0], dtype=torch.int32)
        temp, uni = _host_f32(temperature), _host_f32(uniform)
        self.lib.chibi_ref_sample(_fp(lf), lf.shape[1], lf.shape[0], lf.shape[1], _fp(temp), _fp(uni), _ip(res))
        out.copy_(res.to(out.dtype))
