"""Plain PyTorch restatements of the package's kernels, one per operation, with
the same call signatures as ``chibillm_b200.kernels.ops.CudaKernels``.

Two uses, both in tests only: each CUDA kernel is compared with its
restatement here; and the engine's logic (batching, paging, windows, the
scheduler) is exercised on a machine without a GPU by handing an instance of
:class:`ReferenceKernels` to the runtime in place of the CUDA kernels.  The
arithmetic is 32-bit throughout, results are rounded to the output's type.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


class ReferenceKernels:
    name = "reference"

    def __init__(self):
        self.calls = {}

    def _count(self, name):
        self.calls[name] = self.calls.get(name, 0) + 1

    def check_error_word(self):
        return None

    def embed(self, tokens, table, out):
        self._count("embed")
        out.copy_(table[tokens.long()].float())

    def rmsnorm(self, x, weight, eps, offset, out):
        self._count("rmsnorm")
        xf = x.float()
        n = xf.shape[-1]
        inv = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / n + eps)
        out.copy_(((xf * inv) * (weight.float() + offset)).to(out.dtype))

    def linear_partial(self, x, w, max_splits=0):
        return None

    def linear(self, x, w, out, residual=None, defer=False):
        self._count("linear")
        y = x.float() @ w.float().t()
        if residual is not None:
            y = residual + y
        out.copy_(y.to(out.dtype))

    def qk_norm_rope_append(self, qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq,
                            rotary_dim, eps, norm_offset, positions, seq_of_token, block_table,
                            nq, nkv, d, page_size, seq_rows=None):
        self._count("qk_norm_rope_append")
        T = qkv.shape[0]
        qw, kw = nq * d, nkv * d
        append = k_cache is not None
        q = qkv[:, :qw].float().reshape(T, nq, d)

        def norm(x, w):
            if w is None:
                return x
            inv = torch.rsqrt((x * x).sum(-1, keepdim=True) / d + eps)
            return (x * inv) * (w.float() + norm_offset)

        def rotate(x):
            if not rotary_dim:
                return x
            half = rotary_dim // 2
            angle = positions.float()[:, None] * inv_freq[:half].float()[None, :]
            c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            lo, hi = x[..., :half], x[..., half:rotary_dim]
            return torch.cat([lo * c - hi * s, hi * c + lo * s, x[..., rotary_dim:]], dim=-1)

        q_out.copy_(rotate(norm(q, q_norm_w)).reshape(T, qw).to(q_out.dtype))
        if not append:
            return
        k = rotate(norm(qkv[:, qw:qw + kw].float().reshape(T, nkv, d), k_norm_w))
        v = qkv[:, qw + kw:qw + 2 * kw].float().reshape(T, nkv, d)
        pos = positions.long()
        rows = seq_of_token.long() if seq_rows is None else seq_rows.long()[seq_of_token.long()]
        pages = block_table[rows, pos // page_size].long()
        assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "append outside the pool"
        slots = pos % page_size
        k_cache[pages, :, slots, :] = k.to(k_cache.dtype)
        v_cache[pages, :, slots, :] = v.to(v_cache.dtype)

    def attention(self, q, k_cache, v_cache, out, block_table, q_start, ctx_len, seq_of_token,
                  positions, nq, nkv, d, page_size, scale, window, max_q_len, max_ctx_len, min_q_len=0,
                  seq_rows=None):
        self._count("attention")
        T = q.shape[0]
        group = nq // nkv
        qf = q.float().reshape(T, nq, d)
        res = torch.zeros(T, nq, d, dtype=torch.float32, device=q.device)
        for t in range(T):
            s = int(seq_of_token[t])
            if seq_rows is not None:
                s = int(seq_rows[s])
            p = int(positions[t])
            first = max(0, p - window + 1) if window else 0
            idx = torch.arange(first, p + 1, device=q.device)
            pages = block_table[s, idx // page_size].long()
            assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "attention outside the pool"
            keys = k_cache[pages, :, idx % page_size, :].float()      # [n, nkv, d]
            vals = v_cache[pages, :, idx % page_size, :].float()
            for h in range(nq):
                g = h // group
                sc = (keys[:, g, :] @ qf[t, h]) * scale
                pr = torch.softmax(sc, dim=0)
                res[t, h] = pr @ vals[:, g, :]
        out.copy_(res.reshape(T, nq * d).to(out.dtype))

    def apply_table_updates(self, table, updates, capacity):
        n = int(updates[0])
        assert n <= capacity
        for i in range(n):
            row, index, page = (int(v) for v in updates[1 + 3 * i:4 + 3 * i])
            table[row, index] = page

    def swiglu(self, gate_up, out):
        self._count("swiglu")
        inter = out.shape[1]
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def gather_rows(self, x, rows, out):
        self._count("gather_rows")
        out.copy_(x[rows.long()].to(out.dtype))

    def cast(self, x, out):
        out.copy_(x.reshape(out.shape).to(out.dtype))

    def add_into(self, acc, x):
        acc.add_(x.float().reshape(acc.shape))

    def sample(self, logits, temperature, uniform, out):
        self._count("sample")
        for r in range(logits.shape[0]):
            row = logits[r].float()
            T = float(temperature[r]) if temperature is not None else 0.0
            if not T > 0.0:
                best = row.max()
                out[r] = int(torch.nonzero(row == best)[0, 0])
                continue
            p = torch.exp((row - row.max()) / T).double()
            cdf = torch.cumsum(p, 0)
            target = float(uniform[r]) * float(cdf[-1])
            idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
            out[r] = min(idx, row.numel() - 1)
