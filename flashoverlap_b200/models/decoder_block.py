"""Tensor-parallel decoder block (Llama-style) built on the three fused
operations of the library:

* attention out-projection:  GEMM + all-reduce           (``gemm_allreduce_fused``)
* MLP down-projection:       GEMM + reduce-scatter       (``gemm_reducescatter_fused``,
  the result stays sharded over tokens: sequence parallelism)
* next layer's QKV:          all-gather + GEMM           (``allgather_gemm``)

The reference has no model code; this block is the layer shape its headline
configurations are taken from (hidden 8192, FFN 28672).  ``forward`` runs the
fused kernels, ``forward_reference`` the same math with torch.matmul and
torch.distributed collectives.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class TPDecoderBlock(nn.Module):
    def __init__(self, impl, hidden: int = 8192, ffn: int = 28672, n_heads: int = 64, n_kv_heads: int = 8,
                 eps: float = 1e-5, algo: int = 8, dtype=torch.bfloat16, device=None, seed: int = 0):
        super().__init__()
        self.impl = impl
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        ws = self.world
        assert n_heads % ws == 0 and ffn % ws == 0 and hidden % n_heads == 0
        self.hidden, self.ffn, self.eps, self.algo = hidden, ffn, eps, algo
        self.head_dim = hidden // n_heads
        self.heads = n_heads // ws
        self.kv_heads = max(1, n_kv_heads // ws)
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device="cpu").manual_seed(seed * 1000 + self.rank)

        def w(rows, cols, fan_in):
            return nn.Parameter((torch.randn(rows, cols, generator=g) / fan_in ** 0.5).to(dev, dtype),
                                requires_grad=False)

        qkv_rows = (self.heads + 2 * self.kv_heads) * self.head_dim
        self.w_qkv = w(qkv_rows, hidden, hidden)                    # column-parallel
        self.w_o = w(hidden, self.heads * self.head_dim, hidden)    # row-parallel
        self.w_gate_up = w(2 * ffn // ws, hidden, hidden)           # column-parallel
        self.w_down = w(hidden, ffn // ws, ffn)                     # row-parallel
        self.w_qkv_next = w(qkv_rows, hidden, hidden)               # next layer's QKV
        gn = torch.Generator(device="cpu").manual_seed(seed * 1000 + 999)  # norm weights are replicated
        self.norm_attn = nn.Parameter((1 + 0.1 * torch.randn(hidden, generator=gn)).to(dev, dtype), requires_grad=False)
        self.norm_next = nn.Parameter((1 + 0.1 * torch.randn(hidden, generator=gn)).to(dev, dtype), requires_grad=False)

    # ---- shared pieces ----------------------------------------------------
    def _attention(self, qkv, batch, seq):
        hd, h, kv = self.head_dim, self.heads, self.kv_heads
        q, k, v = qkv.split([h * hd, kv * hd, kv * hd], dim=-1)
        q = q.reshape(batch, seq, h, hd).transpose(1, 2)
        k = k.reshape(batch, seq, kv, hd).transpose(1, 2).repeat_interleave(h // kv, dim=1)
        v = v.reshape(batch, seq, kv, hd).transpose(1, 2).repeat_interleave(h // kv, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return o.transpose(1, 2).reshape(batch * seq, h * hd).contiguous()

    def _mlp_act(self, gu):
        gate, up = gu.chunk(2, dim=-1)
        return (F.silu(gate) * up).contiguous()

    # ---- fused path ---------------------------------------------------------
    @torch.no_grad()
    def forward(self, h_norm, resid, batch, seq):
        """h_norm: normalised block input [tokens, hidden] (replicated), resid: the
        residual stream [tokens, hidden].  Returns (next layer's QKV for all
        tokens [tokens, qkv_rows], new residual shard [tokens/world, hidden])."""
        impl, a = self.impl, self.algo
        T = h_norm.shape[0]
        qkv = torch.empty((T, self.w_qkv.shape[0]), dtype=h_norm.dtype, device=h_norm.device)
        impl.cutlass_gemm(h_norm, self.w_qkv, qkv, self._fit(T, self.w_qkv.shape[0]))
        attn = self._attention(qkv, batch, seq)
        o = impl.gemm_allreduce_fused(attn, self.w_o, None, self.eps, a)          # GEMM + all-reduce
        h2 = resid + o
        m_in = torch.empty_like(h2)
        torch.ops.flashoverlap_op.rmsnorm(h2, m_in, self.norm_attn, self.eps)
        gu = torch.empty((T, self.w_gate_up.shape[0]), dtype=h2.dtype, device=h2.device)
        impl.cutlass_gemm(m_in, self.w_gate_up, gu, self._fit(T, self.w_gate_up.shape[0]))
        act = self._mlp_act(gu)
        rows = T // self.world
        y = torch.empty((rows, self.hidden), dtype=h2.dtype, device=h2.device)
        impl.gemm_reducescatter_fused(act, self.w_down, y, None, self.eps, a, False)  # GEMM + reduce-scatter
        h3 = h2[self.rank * rows:(self.rank + 1) * rows] + y
        n = torch.empty_like(h3)
        torch.ops.flashoverlap_op.rmsnorm(h3, n, self.norm_next, self.eps)
        qkv_next = torch.empty((T, self.w_qkv_next.shape[0]), dtype=h3.dtype, device=h3.device)
        impl.allgather_gemm(n, self.w_qkv_next, qkv_next, self._fit_gather(T, self.w_qkv_next.shape[0]))  # all-gather + GEMM
        return qkv_next, h3

    def _fit(self, M, N):
        """The preferred tile configuration if it divides the shape, else a smaller one."""
        from ..utils.config import ALGO_TILES

        for algo in (self.algo, 3, 0, 1, 2):
            bm, bn, _ = ALGO_TILES[algo]
            if M % bm == 0 and N % bn == 0:
                return algo
        raise ValueError(f"no tile configuration divides {M} x {N}")

    def _fit_gather(self, M, N):
        """Tile configuration of the all-gather GEMM: the gathered rows are consumed
        shard by shard, so the tile is chosen for the tiles ONE shard gives."""
        from ..tune.model import gather_algo_candidates
        from ..utils.config import ALGO_TILES

        if self.world == 1:
            return self._fit(M, N)
        for algo in gather_algo_candidates(M // self.world, N):
            if M % ALGO_TILES[algo][0] == 0:
                return algo
        return self._fit(M, N)

    # ---- PyTorch path -------------------------------------------------------
    @torch.no_grad()
    def forward_reference(self, h_norm, resid, batch, seq):
        T = h_norm.shape[0]
        qkv = h_norm @ self.w_qkv.t()
        attn = self._attention(qkv, batch, seq)
        o = attn @ self.w_o.t()
        if self.world > 1:
            dist.all_reduce(o)
        h2 = resid + o
        m_in = _rms(h2, self.norm_attn, self.eps)
        act = self._mlp_act(m_in @ self.w_gate_up.t())
        part = act @ self.w_down.t()
        rows = T // self.world
        if self.world > 1:
            y = torch.empty((rows, self.hidden), dtype=part.dtype, device=part.device)
            dist.reduce_scatter_tensor(y, part)
        else:
            y = part
        h3 = h2[self.rank * rows:(self.rank + 1) * rows] + y
        n = _rms(h3, self.norm_next, self.eps)
        if self.world > 1:
            full = torch.empty((T, self.hidden), dtype=n.dtype, device=n.device)
            dist.all_gather_into_tensor(full, n.contiguous())
        else:
            full = n
        return full @ self.w_qkv_next.t(), h3
