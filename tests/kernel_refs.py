"""Plain PyTorch float32 references of the CUDA kernels, one per kernel.

Two uses: the ``-m gpu`` tests compare each kernel with its reference at sizes
other than the engine's, and the ``-m "not gpu"`` tests put these functions in
the kernels' place (``patch_ops``) to run the engine's own step function, cache
and batching on the CPU, where only the logic is under test.  They follow the
kernels' signatures in acvram_b200/kernels/ops.py and the rounding points the
kernels document; they are test code, not a second backend of the package.
"""

from __future__ import annotations

import torch


def _r(x: torch.Tensor, dtype) -> torch.Tensor:
    """Round to dtype and come back to float32."""
    return x.to(dtype).to(torch.float32)


def embed(table, tokens, out):
    out.copy_(table[tokens.long()])
    return out


def add_rmsnorm(x, delta, weight, eps, out, rows=None):
    dt = x.dtype
    if rows is None:
        v = x.float()
        if delta is not None:
            v = _r(v + delta.float(), dt)
            x.copy_(v.to(dt))
    else:
        idx = rows.long()
        v = x[idx].float()
        if delta is not None:
            v = _r(v + delta[idx].float(), dt)
    rs = torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_((_r(v * rs, dt) * weight.float()).to(dt))
    return out


def add_bias(out, bias):
    out.copy_((out.float() + bias.float()).to(out.dtype))
    return out


def swiglu(gate_up, out):
    I = out.shape[1]
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    out.copy_((_r(g / (1.0 + torch.exp(-g)), out.dtype) * u).to(out.dtype))
    return out


def _row(table_rows, seq: int) -> int:
    """The row of the block table that belongs to request ``seq`` of the batch."""
    return seq if table_rows is None else int(table_rows[seq])


def table_update(table, triples, n):
    t = triples[:3 * n].view(n, 3).long()
    for row, col, page in t.tolist():
        if 0 <= row < table.shape[0] and 0 <= col < table.shape[1]:
            table[row, col] = page


def qk_norm_rope_append(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos_sin, positions,
                        seq_of_token, block_table, k_pages, v_pages, table_rows=None):
    T = qkv.shape[0]
    NH, NKV, D = num_heads, num_kv_heads, head_dim
    dt = qkv.dtype
    q = qkv[:, :NH * D].float().view(T, NH, D)
    k = qkv[:, NH * D:(NH + NKV) * D].float().view(T, NKV, D)
    v = qkv[:, (NH + NKV) * D:].float().view(T, NKV, D)
    pos = positions.long()

    def norm_rot(x, w):
        if w is not None:
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        if cos_sin is not None:
            rot = cos_sin.shape[1]
            half = rot // 2
            c = cos_sin[pos, :half].float()[:, None, :]
            s = cos_sin[pos, half:].float()[:, None, :]
            a, b = x[..., :half], x[..., half:rot]
            x = torch.cat((a * c - b * s, b * c + a * s, x[..., rot:]), dim=-1)
        return x

    q = norm_rot(q, q_weight)
    k = norm_rot(k, k_weight)
    qkv[:, :NH * D] = q.reshape(T, NH * D).to(dt)
    if k_pages is None:
        qkv[:, NH * D:(NH + NKV) * D] = k.reshape(T, NKV * D).to(dt)
        return
    page = k_pages.shape[2]
    for t in range(T):
        pg = int(block_table[_row(table_rows, int(seq_of_token[t])), int(pos[t]) // page])
        if pg < 0:
            continue
        k_pages[pg, :, int(pos[t]) % page] = k[t].to(dt)
        v_pages[pg, :, int(pos[t]) % page] = v[t].to(dt)


def attention_generic(q, out, k_pages, v_pages, positions, seq_of_token, block_table, num_heads, num_kv_heads,
                      head_dim, scale, window=0, table_rows=None):
    T = q.shape[0]
    NH, NKV, D = num_heads, num_kv_heads, head_dim
    page = k_pages.shape[2]
    rep = NH // NKV
    for t in range(T):
        p = int(positions[t])
        seq = int(seq_of_token[t])
        lo = max(0, p - window + 1) if window > 0 else 0
        js = torch.arange(lo, p + 1, device=q.device)
        pages = block_table[_row(table_rows, seq)].long()[js // page]
        keep = pages >= 0
        js, pages = js[keep], pages[keep]
        kk = k_pages[pages, :, js % page].float()      # [n, NKV, D]
        vv = v_pages[pages, :, js % page].float()
        qq = q[t, :NH * D].float().view(NH, D)
        kk = kk.repeat_interleave(rep, dim=1)
        vv = vv.repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", qq, kk) * scale
        pr = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", pr, vv).reshape(NH * D).to(out.dtype)
    return out


def attention(qkv, out, k_pages, v_pages, ctx, block_table, num_heads, num_kv_heads, head_dim, scale, window=0, work=None):
    return attention_generic(qkv, out, k_pages, v_pages, ctx.positions, ctx.seq_of_token, block_table, num_heads,
                             num_kv_heads, head_dim, scale, window, table_rows=getattr(ctx, "table_rows", None))


def gemm_simt(a, w, out):
    out.copy_((a.float() @ w.float().T).to(out.dtype))
    return out


def linear_bf16(x, w, out):
    return gemm_simt(x, w, out)


def linear_bf16_f32out(x, w, out):
    return gemm_simt(x, w, out)


def argmax(logits, out):
    out.copy_(logits.argmax(-1).to(out.dtype))
    return out


PATCHABLE = ["embed", "add_rmsnorm", "swiglu", "add_bias", "table_update", "qk_norm_rope_append", "attention_generic", "attention", "gemm_simt",
             "linear_bf16", "linear_bf16_f32out", "argmax"]


def patch_ops(monkeypatch) -> None:
    """Put the references in the kernels' place (CPU logic tests only)."""
    import sys

    from acvram_b200.kernels import ops
    me = sys.modules[__name__]
    for name in PATCHABLE:
        monkeypatch.setattr(ops, name, getattr(me, name))
