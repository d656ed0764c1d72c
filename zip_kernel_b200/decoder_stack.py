"""Decoder-stack harness: a random-init Llama-3-8B-architecture decoder whose
linears are W4A4 containers served by this library.

The reference has no W4A4 decoder stack (its layer harness is a single BF16
Qwen3 layer used for per-op timing, ``bench/layer/qwen3_layer_bf16.py:129-241``,
with the fused four-projection enumeration of ``bench/configs/qwen3_shapes.py:96-107``);
this harness runs the workload its configuration list names: ``n_layers`` layers of
hidden 4096, 32 query / 8 KV heads, FFN 14336, vocabulary 128256, the q/k/v and
gate/up projections fused into one linear each (4 W4A4 GEMMs per layer, 7
projections), fp16 RMSNorm / rotary embedding / attention through PyTorch, batch
32, a 1024-token prefill and 128 decode steps.  The decode step is captured once
as a CUDA graph and replayed.  Weights are seeded random: no checkpoint is read.

    python -m zip_kernel_b200.decoder_stack [--layers 32] [--batch 32] [--prefill 1024] [--decode 128]

prints one JSON line with prefill and decode tokens per second.
"""

from __future__ import annotations

import argparse
import json
import math
import time
from dataclasses import dataclass
from typing import List

import torch
import torch.nn.functional as F

from . import _lib, synth
from .pack_utils import V9WeightContainer
from .v9_linear import (prepare_for_prefill, v9_linear_forward, v9_linear_forward_rmsnorm,
                        v9_linear_forward_silu_mul)


@dataclass
class StackConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    density: float = 0.05          # residual blocks

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads


class Layer:
    def __init__(self, cfg: StackConfig, protos, device, prepared: bool):
        # distinct device copies per layer: a layer never finds its weights in L2 because another layer left them there
        self.qkv, self.o, self.gate_up, self.down = (p.to(device) for p in protos)
        if prepared:
            # prompt processing runs the fp8 instantiation of the tensor-core kernel on weights widened once
            # (2 x the packed bytes on top); decode steps keep streaming the packed arrays
            for W in (self.qkv, self.o, self.gate_up, self.down):
                prepare_for_prefill(W)
        self.norm1 = torch.ones(cfg.hidden, dtype=torch.float16, device=device)
        self.norm2 = torch.ones(cfg.hidden, dtype=torch.float16, device=device)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.float16) * w


def rope_tables(cfg: StackConfig, max_pos: int, device):
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device, dtype=torch.float32) / cfg.head_dim))
    ang = torch.outer(torch.arange(max_pos, device=device, dtype=torch.float32), inv)
    return ang.cos().to(torch.float16), ang.sin().to(torch.float16)       # (max_pos, head_dim / 2)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (B, S, H, D); cos/sin (S, D/2) or (B, S, D/2)."""
    x1, x2 = x[..., ::2], x[..., 1::2]
    c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
    if c.dim() == 3:
        c, s = c.unsqueeze(0), s.unsqueeze(0)
    return torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1).flatten(-2)


class DecoderStack:
    """Weights, KV cache and the two phases (prefill of a prompt batch, one decode step)."""

    def __init__(self, cfg: StackConfig, batch: int, max_len: int, device, seed: int = 0, prepared: bool = True,
                 fused_seams: bool = True):
        self.cfg, self.batch, self.max_len, self.device = cfg, batch, max_len, device
        # fused_seams: RMSNorm and SiLU * mul run inside the quantisation launch of the linear they feed
        # (v9_linear_forward_rmsnorm / _silu_mul) instead of as separate PyTorch kernels
        self.fused_seams = fused_seams
        h, kv = cfg.hidden, cfg.n_kv_heads * cfg.head_dim
        shapes = [(h, h + 2 * kv), (h, h), (h, 2 * cfg.ffn), (cfg.ffn, h)]             # (d_in, d_out)
        protos: List[V9WeightContainer] = [
            synth.make_container(n, k, cfg.density, seed=synth.shape_seed(seed, k, n)) for k, n in shapes]
        for W in protos:
            # the synthetic scales (U(0.001, 0.051) on codes of standard deviation 4.6) give outputs of
            # standard deviation ~0.15 * sqrt(K) for unit inputs; bring every projection to ~0.5 so that
            # the residual stream of a deep random stack stays inside fp16
            W.scale_u4 = (W.scale_u4.float() * (0.5 / (0.15 * math.sqrt(W.d_in)))).to(torch.float16)
        self.layers = [Layer(cfg, protos, device, prepared) for _ in range(cfg.n_layers)]
        g = torch.Generator().manual_seed(seed + 1)
        self.embed = (torch.randn(cfg.vocab, h, generator=g) * 0.02).to(torch.float16).to(device)
        self.lm_head = (torch.randn(cfg.vocab, h, generator=g) * 0.02).to(torch.float16).to(device)
        self.final_norm = torch.ones(h, dtype=torch.float16, device=device)
        self.cos, self.sin = rope_tables(cfg, max_len, device)
        self.k_cache = torch.zeros(cfg.n_layers, batch, cfg.n_kv_heads, max_len, cfg.head_dim, dtype=torch.float16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)

    # ---- one layer on hidden states x (B, S, hidden) whose tokens sit at positions pos .. pos + S - 1
    def _layer(self, li: int, x: torch.Tensor, pos, S: int, attend_len) -> torch.Tensor:
        cfg, L = self.cfg, self.layers[li]
        B = x.shape[0]
        hd, nh, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        if self.fused_seams:
            qkv = v9_linear_forward_rmsnorm(x, L.norm1, cfg.rms_eps, L.qkv)
        else:
            qkv = v9_linear_forward(rms_norm(x, L.norm1, cfg.rms_eps), L.qkv)
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        q = q.view(B, S, nh, hd)
        k = k.view(B, S, nkv, hd)
        v = v.view(B, S, nkv, hd)
        if isinstance(pos, int):
            cos, sin = self.cos[pos:pos + S], self.sin[pos:pos + S]
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            self.k_cache[li, :, :, pos:pos + S] = k.transpose(1, 2)
            self.v_cache[li, :, :, pos:pos + S] = v.transpose(1, 2)
            att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                 is_causal=True, enable_gqa=True)
        else:
            # decode under a CUDA graph: the position is a device tensor, the cache is
            # written by index and attention masks the tail of the preallocated cache
            cos, sin = self.cos.index_select(0, pos), self.sin.index_select(0, pos)        # (1, hd/2)
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            self.k_cache[li].index_copy_(2, pos, k.transpose(1, 2))
            self.v_cache[li].index_copy_(2, pos, v.transpose(1, 2))
            keys, vals = self.k_cache[li, :, :, :attend_len], self.v_cache[li, :, :, :attend_len]
            mask = (torch.arange(attend_len, device=x.device) <= pos).view(1, 1, 1, attend_len)
            att = F.scaled_dot_product_attention(q.transpose(1, 2), keys, vals, attn_mask=mask, enable_gqa=True)
        x = x + v9_linear_forward(att.transpose(1, 2).reshape(B, S, nh * hd), L.o)
        if self.fused_seams:
            gu = v9_linear_forward_rmsnorm(x, L.norm2, cfg.rms_eps, L.gate_up)
            return x + v9_linear_forward_silu_mul(gu, L.down)
        gu = v9_linear_forward(rms_norm(x, L.norm2, cfg.rms_eps), L.gate_up)
        gate, up = gu.split(cfg.ffn, dim=-1)
        return x + v9_linear_forward(F.silu(gate) * up, L.down)

    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens (B, S) -> next-token ids (B,)"""
        S = tokens.shape[1]
        x = self.embed[tokens]
        for li in range(self.cfg.n_layers):
            x = self._layer(li, x, 0, S, None)
        logits = rms_norm(x[:, -1], self.final_norm, self.cfg.rms_eps) @ self.lm_head.t()
        return logits.argmax(-1)

    def decode_step(self, tokens: torch.Tensor, pos: torch.Tensor, attend_len: int) -> torch.Tensor:
        """tokens (B,), pos (1,) int64 device tensor -> next-token ids (B,)"""
        x = self.embed[tokens].unsqueeze(1)
        for li in range(self.cfg.n_layers):
            x = self._layer(li, x, pos, 1, attend_len)
        logits = rms_norm(x[:, 0], self.final_norm, self.cfg.rms_eps) @ self.lm_head.t()
        return logits.argmax(-1)


def run(cfg: StackConfig, batch: int, prefill_len: int, decode_steps: int, device, use_graph: bool = True, seed: int = 0,
        prepared: bool = True, fused_seams: bool = True):
    max_len = prefill_len + decode_steps
    stack = DecoderStack(cfg, batch, max_len, device, seed, prepared, fused_seams)
    g = torch.Generator().manual_seed(seed + 2)
    prompt = torch.randint(0, cfg.vocab, (batch, prefill_len), generator=g).to(device)

    with torch.no_grad():
        stack.prefill(prompt[:, : min(prefill_len, 128)])      # warm-up: sizes the library's scratch for the tensor-core path
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        nxt = stack.prefill(prompt)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0

        pos = torch.tensor([prefill_len], dtype=torch.int64, device=device)
        tok = nxt.clone()
        out = torch.empty_like(tok)
        produced = [nxt.clone()]
        graph = None
        scratch = _lib.WorkspaceHolder()      # the captured step writes scratch of its own, alive as long as the graph
        if use_graph:
            side = torch.cuda.Stream()
            with _lib.use_workspace(scratch), torch.cuda.stream(side):
                stack.decode_step(tok, pos, max_len)           # warm-up on the capture stream (scratch is per stream)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    out.copy_(stack.decode_step(tok, pos, max_len))
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(decode_steps):
            if graph is not None:
                graph.replay()
            else:
                out.copy_(stack.decode_step(tok, pos, max_len))
            tok.copy_(out)
            pos += 1
            produced.append(out.clone())
        e1.record()
        torch.cuda.synchronize()
        t_decode = e0.elapsed_time(e1) / 1e3
    return {
        "metric": "decoder_stack_decode_tokens_per_s", "value": batch * decode_steps / t_decode, "unit": "tok/s",
        "prefill_tokens_per_s": batch * prefill_len / t_prefill, "ms_per_decode_step": t_decode / decode_steps * 1e3,
        "prefill_s": t_prefill, "data": "synthetic (seeded random weights and token ids)",
        "config": {"layers": cfg.n_layers, "hidden": cfg.hidden, "heads": f"{cfg.n_heads}/{cfg.n_kv_heads}", "ffn": cfg.ffn,
                   "vocab": cfg.vocab, "batch": batch, "prefill": prefill_len, "decode_steps": decode_steps,
                   "w4a4_linears_per_layer": "qkv, o, gate_up, down (7 projections)", "residual_density": cfg.density,
                   "decode_step": "CUDA graph" if use_graph else "eager",
                   "prefill_weights": "prepared e4m3 copy" if prepared else "packed",
                   "seams": "RMSNorm and SiLU*mul fused into the quantisation launches" if fused_seams else "PyTorch RMSNorm / SiLU*mul"},
        "last_tokens": [int(t) for t in produced[-1][:4].tolist()],
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prefill", type=int, default=1024)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-prepared", action="store_true", help="prompt processing on the packed weights")
    ap.add_argument("--no-fused-seams", action="store_true", help="RMSNorm and SiLU*mul as separate PyTorch kernels")
    a = ap.parse_args()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    res = run(StackConfig(n_layers=a.layers), a.batch, a.prefill, a.decode, device, use_graph=not a.no_graph,
              prepared=not a.no_prepared, fused_seams=not a.no_fused_seams)
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
