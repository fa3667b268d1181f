"""The caller of the fused epilogue: a tensor-parallel Llama-style decoder for inference.

Mirrors the structure of the reference's ``model/transformer_model.py:397-811`` (``ModelArgs``,
``Attention`` with grouped-query heads, interleaved-pair RoPE and a KV cache, SwiGLU
``FeedForward``, pre-norm ``TransformerBlock``) and ``model/tensor_parallel.py:34-123``
(column-parallel ``wq/wk/wv/w1/w3``, row-parallel ``wo/w2``), with the one change the fused
operator exists for: a row-parallel projection returns its *partial* sums, and

    h, normed, scale = env.allreduce_add_rms_fused(partial, h, next_norm.weight, eps, fp8_out)

replaces ``reduce_from_tensor_parallel_region`` + ``x + ...`` + the following ``RMSNorm``
(``tensor_parallel.py:117-118``, ``transformer_model.py:610-618``) at both sites of every
layer.  With ``fp8=True`` the normalised activations leave the operator as FP8-e4m3 with one
scale per token, and the column-parallel projections that consume them run as FP8 GEMMs with
row-wise scales: for decode batches this library's own weight-streaming kernel (``gpuk_b200.fp8_linear``,
``csrc/fp8_linear.cu``) where it is the faster one on B200 (up to 16 tokens, or up to 32 tokens and at most 4096
output channels per shard; measured in ``bench.py --case fp8_linear``), otherwise ``torch._scaled_mm`` (a library
GEMM; ``own_fp8_gemm=False`` uses it everywhere).  Both give the same results to within one bf16 step.

``fused=False`` runs the reference arrangement on the same weights -- NCCL ``all_reduce``, then
add, RMSNorm (and quantisation) as separate PyTorch operators -- and is the comparison arm.

Fix-ups relative to the reference, which cannot run with more than one rank as it stands
(``WorkerProc.__call__`` raises, ``:788-789``): the KV cache holds this rank's KV heads only
(the reference sizes it with the global count, ``:674``), weights are random-initialised per
shard on the device, and nothing is compiled or traced.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F


@dataclass
class DecoderArgs:
    """Subset of the reference's ``ModelArgs`` (``transformer_model.py:419-443``) a dense decoder needs."""
    dim: int = 8192
    n_layers: int = 4
    n_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 28672
    vocab_size: int = 32768
    max_seq_len: int = 2304
    norm_eps: float = 1e-6
    rope_theta: float = 500000.0
    dtype: torch.dtype = torch.bfloat16


def _shard_rows(master: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel shard: rows [rank*n/world, (rank+1)*n/world) of a [out, in] weight (``tensor_parallel.py:24-30``)."""
    n = master.shape[0] // world
    return master[rank * n:(rank + 1) * n].contiguous()


def _shard_cols(master: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Row-parallel shard: columns of a [out, in] weight."""
    n = master.shape[1] // world
    return master[:, rank * n:(rank + 1) * n].contiguous()


def _xavier(out_f: int, in_f: int, gen: torch.Generator, device, dtype) -> torch.Tensor:
    std = math.sqrt(2.0 / (in_f + out_f))     # init.xavier_normal_ on the full matrix (tensor_parallel.py:62-67)
    return (torch.randn(out_f, in_f, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


class _Linear:
    """y = x @ W^T for one shard, in the activation dtype or as an FP8 GEMM with row-wise scales."""

    def __init__(self, weight: torch.Tensor, fp8: bool, own_gemm: bool = True):
        self.weight = weight                                  # [out_local, in]
        self.fp8 = fp8
        self.own_gemm = own_gemm                              # decode batches: this library's weight-streaming FP8 kernel
        self.w_packed = None                                  # ... its blocked copy of the weights, made at first use
        if fp8:
            amax = weight.float().abs().amax(dim=1, keepdim=True).clamp_(min=1e-12)
            self.w_scale = (amax / 448.0).t().contiguous()    # [1, out_local] fp32, one scale per output channel
            self.w_q = (weight.float() / amax * 448.0).clamp_(-448, 448).to(torch.float8_e4m3fn)   # [out, in] row-major

    def __call__(self, x: torch.Tensor, x_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.fp8 and x.dtype == torch.float8_e4m3fn:
            if self.own_gemm and x.is_cuda:
                import gpuk_b200 as gpuk
                # measured on B200 (bench.py --case fp8_linear): faster than the library GEMM up to 16 tokens at every
                # shape of the decoder, and up to 32 tokens where the shard has at most 4096 output channels
                m, n = x.shape[0], self.w_q.shape[0]
                if (gpuk.fp8_linear_supported(m, n, self.w_q.shape[1]) and (m <= 16 or n <= 4096)
                        and self.weight.dtype == torch.bfloat16):
                    if self.w_packed is None:
                        self.w_packed = gpuk.fp8_pack_weight(self.w_q)
                    return gpuk.fp8_linear(x, x_scale, self.w_packed, self.w_scale, packed=True)
            return torch._scaled_mm(x, self.w_q.t(), scale_a=x_scale, scale_b=self.w_scale, out_dtype=self.weight.dtype)
        return F.linear(x, self.weight)


class TPDecoder:
    """Random-initialised decoder, sharded over the ranks of ``env``'s group; inference only."""

    def __init__(self, args: DecoderArgs, env, *, device, fused: bool = True, fp8: bool = True, seed: int = 1234,
                 master_init: bool = False, max_batch: int = 32, own_fp8_gemm: bool = True):
        self.args, self.env, self.device, self.fused, self.fp8 = args, env, torch.device(device), fused, fp8
        self.rank, self.world = env.rank, env.world_size
        a, w, r = args, self.world, self.rank
        assert a.n_heads % w == 0 and a.n_kv_heads % w == 0 and a.ffn_dim % w == 0, "heads and FFN must divide over the ranks"
        self.h_local, self.kv_local = a.n_heads // w, a.n_kv_heads // w
        hd = a.head_dim

        def make(out_f, in_f, tag, split):
            """One weight shard.  master_init draws the full matrix (identical on all ranks, as the
            reference does on the CPU) and slices it; otherwise the shard is drawn directly."""
            if master_init:
                g = torch.Generator(device="cpu").manual_seed(seed * 1000 + tag)
                m = _xavier(out_f, in_f, g, "cpu", a.dtype)
                s = _shard_rows(m, r, w) if split == "rows" else (_shard_cols(m, r, w) if split == "cols" else m)
                return s.to(self.device)
            g = torch.Generator(device=self.device).manual_seed(seed * 1000 + tag * 16 + (r if split else 0))
            so, si = (out_f // w, in_f) if split == "rows" else ((out_f, in_f // w) if split == "cols" else (out_f, in_f))
            std_w = _xavier(so, si, g, self.device, torch.float32) * (math.sqrt(so + si) / math.sqrt(out_f + in_f))
            return std_w.to(a.dtype)

        self.tok_embeddings = make(a.vocab_size, a.dim, 1, None)
        self.layers: List[dict] = []
        for li in range(a.n_layers):
            t = 100 * (li + 1)
            wq = make(a.n_heads * hd, a.dim, t + 1, "rows")
            wk = make(a.n_kv_heads * hd, a.dim, t + 2, "rows")
            wv = make(a.n_kv_heads * hd, a.dim, t + 3, "rows")
            w1 = make(a.ffn_dim, a.dim, t + 5, "rows")
            w3 = make(a.ffn_dim, a.dim, t + 6, "rows")
            norm_gen = torch.Generator(device="cpu").manual_seed(seed * 1000 + t + 8)
            self.layers.append({
                # one GEMM for q|k|v and one for w1|w3: they share their input
                "wqkv": _Linear(torch.cat([wq, wk, wv], 0), fp8, own_fp8_gemm),
                "wo": _Linear(make(a.dim, a.n_heads * hd, t + 4, "cols"), False),
                "w13": _Linear(torch.cat([w1, w3], 0), fp8, own_fp8_gemm),
                "w2": _Linear(make(a.dim, a.ffn_dim, t + 7, "cols"), False),
                "attention_norm": (1 + 0.1 * torch.randn(a.dim, generator=norm_gen)).to(a.dtype).to(self.device),
                "ffn_norm": (1 + 0.1 * torch.randn(a.dim, generator=norm_gen)).to(a.dtype).to(self.device),
                "k_cache": torch.zeros(max_batch, self.kv_local, a.max_seq_len, hd, dtype=a.dtype, device=self.device),
                "v_cache": torch.zeros(max_batch, self.kv_local, a.max_seq_len, hd, dtype=a.dtype, device=self.device),
            })
        norm_gen = torch.Generator(device="cpu").manual_seed(seed * 1000 + 9)
        self.norm = (1 + 0.1 * torch.randn(a.dim, generator=norm_gen)).to(a.dtype).to(self.device)
        self.output = _Linear(make(a.vocab_size, a.dim, 2, "rows"), fp8, own_fp8_gemm)
        inv = 1.0 / (a.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.int64).float() / hd))   # :497-502
        freqs = torch.outer(torch.arange(a.max_seq_len * 2, dtype=torch.float32), inv)
        self.cos, self.sin = freqs.cos().to(self.device), freqs.sin().to(self.device)
        self._zeros = {}

    # ------------------------------------------------------------------------------------
    def fill_kv_cache(self, upto: int, seed: int = 7) -> None:
        """Seeded N(0,1) keys and values for positions [0, upto): stands in for a prefill."""
        for li, layer in enumerate(self.layers):
            g = torch.Generator(device=self.device).manual_seed(seed * 100 + li * 16 + self.rank)
            for name in ("k_cache", "v_cache"):
                c = layer[name]
                c[:, :, :upto] = torch.randn(c.shape[0], c.shape[1], upto, c.shape[3], generator=g, device=self.device,
                                             dtype=torch.float32).to(c.dtype)

    def _rope(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """Interleaved pairs in, halves out (``transformer_model.py:504-519``, rope_interval_split)."""
        x1, x2 = x[..., 0::2], x[..., 1::2]
        cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).type_as(x)

    def _norm_only(self, h: torch.Tensor, weight: torch.Tensor):
        """RMSNorm (+ FP8) of the embeddings before the first layer: the fused operator with a
        zero residual on this rank alone."""
        if self.fused:
            z = self._zeros.get(h.shape)
            if z is None:
                z = self._zeros[h.shape] = torch.zeros_like(h)
            import gpuk_b200 as gpuk
            residual_out = torch.empty_like(h)
            if self.fp8:
                normed = torch.empty(h.shape, dtype=torch.float8_e4m3fn, device=h.device)
                scale = torch.empty(h.shape[0], 1, dtype=torch.float32, device=h.device)
                gpuk.allreduce_rms(0, h, z, weight, residual_out, normed, scale, self.args.norm_eps, 3)
                return normed, scale
            normed = torch.empty_like(h)
            scale = torch.empty(1, dtype=torch.float32, device=h.device)
            gpuk.allreduce_rms(0, h, z, weight, residual_out, normed, scale, self.args.norm_eps, 0)
            return normed, None
        return self._unfused_norm(h, weight)

    def _unfused_norm(self, h, weight):
        v = h.float().pow(2).mean(-1, keepdim=True)
        n = weight * (h * torch.rsqrt(v + self.args.norm_eps)).to(h.dtype)
        if not self.fp8:
            return n, None
        scale = n.float().abs().amax(dim=-1, keepdim=True) / 448.0
        return (n.float() / scale).clamp_(-448, 448).to(torch.float8_e4m3fn), scale

    def _reduce_add_norm(self, partial, h, weight) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
        """all-reduce(partial) + h -> new h; RMSNorm(new h) * weight (-> FP8) -> input of the next projections."""
        if self.fused:
            h, normed, scale = self.env.allreduce_add_rms_fused(partial, h, weight, self.args.norm_eps, self.fp8)
            return h, normed, (scale if self.fp8 else None)
        if self.world > 1:
            dist.all_reduce(partial, group=self.env.group)       # tensor_parallel.py:118
        h = h + partial                                          # transformer_model.py:611,617
        normed, scale = self._unfused_norm(h, weight)            # :466-471
        return h, normed, scale

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, input_pos: torch.Tensor, cache_len: Optional[int] = None) -> torch.Tensor:
        """tokens [b, t] at positions input_pos [t] (KV cache updated in place) -> logits [b, t, vocab/world]
        of this rank's vocabulary shard.  cache_len = last position + 1; pass it to avoid a device read."""
        a = self.args
        b, t = tokens.shape
        hd = a.head_dim
        h = F.embedding(tokens, self.tok_embeddings).view(b * t, a.dim)
        cos, sin = self.cos[input_pos], self.sin[input_pos]
        last = int(input_pos[-1]) + 1 if cache_len is None else cache_len
        mask = None
        if t > 1:
            mask = (torch.arange(last, device=self.device)[None, :] <= input_pos[:, None])[None, None]
        normed, scale = self._norm_only(h, self.layers[0]["attention_norm"])
        for li, layer in enumerate(self.layers):
            qkv = layer["wqkv"](normed, scale).view(b, t, self.h_local + 2 * self.kv_local, hd)
            q, k, v = qkv.split([self.h_local, self.kv_local, self.kv_local], dim=2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            layer["k_cache"][:b, :, input_pos] = k.transpose(1, 2)
            layer["v_cache"][:b, :, input_pos] = v.transpose(1, 2)
            att = F.scaled_dot_product_attention(q.transpose(1, 2), layer["k_cache"][:b, :, :last], layer["v_cache"][:b, :, :last],
                                                 attn_mask=mask, enable_gqa=True)
            partial = layer["wo"](att.transpose(1, 2).reshape(b * t, self.h_local * hd))
            h, normed, scale = self._reduce_add_norm(partial, h, layer["ffn_norm"])
            g13 = layer["w13"](normed, scale)
            f1, f3 = g13.split(a.ffn_dim // self.world, dim=-1)
            partial = layer["w2"](F.silu(f1) * f3)
            nxt = self.layers[li + 1]["attention_norm"] if li + 1 < a.n_layers else self.norm
            h, normed, scale = self._reduce_add_norm(partial, h, nxt)
        return self.output(normed, scale).view(b, t, -1)
