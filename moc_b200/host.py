"""A LLaMA-style decoder host for the B200 MoC FFN plugin.

The reference builds its models with ``moc/model.py`` (``LLaMAModel``: token embedding, pre-norm blocks of
RoPE causal self-attention and a swappable FFN, final RMSNorm, LM head, shifted cross-entropy loss;
model.py:19-149) on the presets of ``moc/config.py:40-69``. On a machine that has the reference checkout the
plugin drops into that host through ``moc_b200.install_into``. This module is the stand-in for machines that
do not have it (the end-to-end benchmarks): the same architecture, the same parameter names and shapes, so
that a reference ``state_dict`` loads unchanged, written on PyTorch's own ops (``scaled_dot_product_attention``,
``cross_entropy``) with the FFN of every block built by ``moc_b200.build_ffn``.

It also carries the decode loop of the reference's end-to-end decode benchmark (static key/value cache, one
token per step, benchmarks/inference/benchmark_decode.py:127-194) with a batch dimension.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from .ffn import build_ffn
from .inference import InferenceMoCSwiGLUFFN


@dataclass
class HostConfig:
    """Same fields and defaults as the reference's MoCConfig (moc/config.py:12-38)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    vocab_size: int = 32000
    max_seq_len: int = 256
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    k: Optional[int] = None

    def __post_init__(self):
        if self.hidden_size % self.num_attention_heads != 0:
            raise ValueError(f"hidden_size ({self.hidden_size}) must be divisible by "
                             f"num_attention_heads ({self.num_attention_heads})")
        if self.k is None:
            self.k = self.hidden_size // 2
        if self.k > self.intermediate_size:
            raise ValueError(f"k ({self.k}) must not exceed intermediate_size ({self.intermediate_size})")


# the model families of moc/config.py:40-69
PRESETS = {
    "60m": dict(hidden_size=512, intermediate_size=1376, num_hidden_layers=8, num_attention_heads=8, k=256),
    "130m": dict(hidden_size=768, intermediate_size=2048, num_hidden_layers=12, num_attention_heads=12, k=384),
    "350m": dict(hidden_size=1024, intermediate_size=2736, num_hidden_layers=24, num_attention_heads=16, k=512),
    "1b": dict(hidden_size=2048, intermediate_size=5461, num_hidden_layers=24, num_attention_heads=32, k=1024),
}


def get_config(preset: str, **overrides) -> HostConfig:
    if preset not in PRESETS:
        raise ValueError(f"Unknown preset '{preset}'. Available: {list(PRESETS.keys())}")
    return HostConfig(**{**PRESETS[preset], **overrides})


class RMSNorm(nn.Module):
    """Root-mean-square norm with the reduction in fp32 (model.py:19-27)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + self.eps)
        return (xf * inv).to(x.dtype) * self.weight


def rope_tables(head_dim: int, positions: int, theta: float):
    """cos / sin of position * theta^(-2i / head_dim), [positions, head_dim / 2] (model.py:30-34)."""
    inv_freq = theta ** (-torch.arange(0, head_dim, 2).float() / head_dim)
    angle = torch.arange(positions).float()[:, None] * inv_freq[None, :]
    return angle.cos(), angle.sin()


def rotate_pairs(x, cos, sin):
    """Rotary embedding on interleaved (even, odd) pairs of the last dimension (model.py:37-43).
    x: [batch, heads, T, head_dim]; cos, sin: [T, head_dim / 2]."""
    even, odd = x[..., 0::2], x[..., 1::2]
    out = torch.stack((even * cos - odd * sin, even * sin + odd * cos), dim=-1)
    return out.flatten(-2)


class SelfAttention(nn.Module):
    """Multi-head causal self-attention with one fused QKV projection (model.py:46-71)."""

    def __init__(self, cfg: HostConfig):
        super().__init__()
        d = cfg.hidden_size
        self.num_heads = cfg.num_attention_heads
        self.head_dim = d // self.num_heads
        self.qkv_proj = nn.Linear(d, 3 * d, bias=False)
        self.out_proj = nn.Linear(d, d, bias=False)
        cos, sin = rope_tables(self.head_dim, cfg.max_seq_len, cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def _qkv(self, x, first_pos: int):
        b, t, _ = x.shape
        qkv = self.qkv_proj(x).view(b, t, 3, self.num_heads, self.head_dim)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))      # [b, heads, t, head_dim]
        cos = self.rope_cos[first_pos:first_pos + t].to(x.dtype)
        sin = self.rope_sin[first_pos:first_pos + t].to(x.dtype)
        return rotate_pairs(q, cos, sin), rotate_pairs(k, cos, sin), v

    def forward(self, x):
        b, t, c = x.shape
        q, k, v = self._qkv(x, 0)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.out_proj(y.transpose(1, 2).reshape(b, t, c))

    def forward_step(self, x, cache_k, cache_v, pos):
        """One new position per row with the position held in a device tensor (`pos`: int64 [1]), so that the call
        has static shapes and can be captured in a CUDA graph: the rotary tables and the cache slot are indexed by
        `pos`, attention runs over the whole cache under a mask of the positions <= pos."""
        b, t, c = x.shape          # t == 1
        qkv = self.qkv_proj(x).view(b, 1, 3, self.num_heads, self.head_dim)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        cos = self.rope_cos.index_select(0, pos).to(x.dtype)
        sin = self.rope_sin.index_select(0, pos).to(x.dtype)
        q, k = rotate_pairs(q, cos, sin), rotate_pairs(k, cos, sin)
        cache_k.index_copy_(2, pos, k)
        cache_v.index_copy_(2, pos, v)
        seen = torch.arange(cache_k.shape[2], device=x.device) <= pos          # [T_max]
        y = F.scaled_dot_product_attention(q, cache_k, cache_v, attn_mask=seen[None, None, None, :])
        return self.out_proj(y.transpose(1, 2).reshape(b, 1, c))

    def forward_cached(self, x, cache_k, cache_v, first_pos: int):
        """x: [b, t, d] for positions first_pos .. first_pos + t - 1; the caches [b, heads, T_max, head_dim] are
        updated in place and attended up to the last new position."""
        b, t, c = x.shape
        q, k, v = self._qkv(x, first_pos)
        cache_k[:, :, first_pos:first_pos + t] = k
        cache_v[:, :, first_pos:first_pos + t] = v
        end = first_pos + t
        if t == 1:
            y = F.scaled_dot_product_attention(q, cache_k[:, :, :end], cache_v[:, :, :end])
        else:
            # prompt: causal inside the new positions, full view of the cached prefix
            mask = torch.ones(t, end, dtype=torch.bool, device=x.device).tril(diagonal=first_pos)
            y = F.scaled_dot_product_attention(q, cache_k[:, :, :end], cache_v[:, :, :end], attn_mask=mask)
        return self.out_proj(y.transpose(1, 2).reshape(b, t, c))


class Block(nn.Module):
    """Pre-norm block: x + attn(norm(x)), then x + ffn(norm(x)) (model.py:74-88)."""

    def __init__(self, cfg: HostConfig, ffn_type: str):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.attn = SelfAttention(cfg)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.ffn = build_ffn(cfg.hidden_size, cfg.intermediate_size, ffn_type=ffn_type, k=cfg.k)

    def forward(self, x):
        x = x + self.attn(self.attn_norm(x))
        return x + self.ffn(self.ffn_norm(x))


_FFN_TYPES = ("dense", "moc", "moc_gcp", "moc_2_8", "moc_post_silu_abs")


class HostLlama(nn.Module):
    """Decoder-only model with the module tree of the reference's LLaMAModel (model.py:91-143): ``tok_emb``,
    ``blocks[i].{attn_norm, attn.{qkv_proj, out_proj}, ffn_norm, ffn.{gate_proj, up_proj, down_proj}}``, ``norm``,
    ``lm_head``. ``forward(input_ids, labels=None)`` returns logits, or (logits, loss) with the loss of position
    t taken against label t + 1 and labels of -100 ignored."""

    def __init__(self, cfg: HostConfig, ffn_type: str = "dense"):
        super().__init__()
        if ffn_type not in _FFN_TYPES:
            raise ValueError("ffn_type must be 'dense', 'moc', 'moc_gcp', 'moc_2_8', "
                             f"or 'moc_post_silu_abs', got {ffn_type!r}")
        self.config = cfg
        self.ffn_type = ffn_type
        self.tok_emb = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.blocks = nn.ModuleList(Block(cfg, ffn_type) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.lm_head = None if cfg.tie_word_embeddings else nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)      # model.py:120-125

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def _logits(self, h):
        h = self.norm(h)
        return h @ self.tok_emb.weight.t() if self.lm_head is None else self.lm_head(h)

    def forward(self, input_ids, labels=None):
        h = self.tok_emb(input_ids)
        for blk in self.blocks:
            h = blk(h)
        logits = self._logits(h)
        if labels is None:
            return logits
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1),
                               ignore_index=-100)
        return logits, loss


def build_model(cfg: HostConfig, ffn_type: str = "dense") -> HostLlama:
    return HostLlama(cfg, ffn_type=ffn_type)


class GreedyDecoder:
    """Greedy generation with a static key/value cache, the loop of the reference's decode benchmark
    (benchmark_decode.py:127-194, :312-385) with a batch dimension. The FFN of every block runs through the decode
    entry points (``InferenceMoCSwiGLUFFN``: global MoC, MoC 2:8 or the dense baseline) on the weights of the
    given model; attention, norms and the LM head are PyTorch ops. One decode step can be captured in a CUDA
    graph (``capture_step``)."""

    def __init__(self, model: HostLlama, batch: int, mode: str = "auto"):
        cfg = model.config
        if model.ffn_type == "moc_post_silu_abs":
            # the decode kernels select on the raw gate; a model trained with Top-K on |SiLU(gate)| would decode
            # with another channel set than its forward pass (the reference has no such decode mode either)
            raise ValueError("GreedyDecoder does not support ffn_type='moc_post_silu_abs'")
        self.model = model
        self.mode = mode
        self.batch = batch
        dev = model.tok_emb.weight.device
        dt = model.tok_emb.weight.dtype
        heads, hd = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
        self.cache_k = [torch.zeros(batch, heads, cfg.max_seq_len, hd, device=dev, dtype=dt) for _ in model.blocks]
        self.cache_v = [torch.zeros_like(c) for c in self.cache_k]
        self.ffn = []
        grouped = model.ffn_type == "moc_2_8"
        for blk in model.blocks:
            f = InferenceMoCSwiGLUFFN(cfg.hidden_size, cfg.intermediate_size, blk.ffn.k if hasattr(blk.ffn, "k") else cfg.k,
                                      *((2, 8) if grouped else (None, None)))
            # the decode modules read the model's own parameters: no copies
            f.gate_proj.weight = blk.ffn.gate_proj.weight
            f.up_proj.weight = blk.ffn.up_proj.weight
            f.down_proj.weight = blk.ffn.down_proj.weight
            f.freeze_for_compile()
            self.ffn.append(f)
        self._graph = None
        self._rope_bf16 = None
        # graph-replayed steps use the library's fused host-step kernels when the model allows (bf16, supported head size)
        self.fused_host_step = True

    @torch.no_grad()
    def _forward(self, ids, first_pos: int):
        m = self.model
        h = m.tok_emb(ids)
        b, t, d = h.shape
        ffn_mode = "dense_baseline" if m.ffn_type == "dense" else self.mode
        for i, blk in enumerate(m.blocks):
            h = h + blk.attn.forward_cached(blk.attn_norm(h), self.cache_k[i], self.cache_v[i], first_pos)
            h = h + self.ffn[i](blk.ffn_norm(h).reshape(b * t, d), mode=ffn_mode).reshape(b, t, d)
        return m._logits(h[:, -1:])[:, 0]

    @torch.no_grad()
    def _step(self, ids, pos):
        """Static-shape decode step: ids [batch, 1], pos int64 [1] on the device. Returns the next token ids."""
        m = self.model
        h = m.tok_emb(ids)
        b, _, d = h.shape
        ffn_mode = "dense_baseline" if m.ffn_type == "dense" else self.mode
        for i, blk in enumerate(m.blocks):
            h = h + blk.attn.forward_step(blk.attn_norm(h), self.cache_k[i], self.cache_v[i], pos)
            h = h + self.ffn[i](blk.ffn_norm(h).reshape(b, d), mode=ffn_mode).reshape(b, 1, d)
        return m._logits(h)[:, 0].argmax(dim=-1)

    def _fused_step_supported(self) -> bool:
        cfg = self.model.config
        hd = cfg.hidden_size // cfg.num_attention_heads
        w = self.model.tok_emb.weight
        return (w.is_cuda and w.dtype == torch.bfloat16 and cfg.hidden_size % 8 == 0 and hd in (8, 16, 32, 64, 128)
                and cfg.max_seq_len <= 11000 and _lib.exported("moc_host_attn_step"))

    @torch.no_grad()
    def _step_fused(self, ids, pos):
        """The same step as _step with the operations around the projections done by the library's host-step
        kernels (moc_host_rmsnorm, moc_host_rope_cache, moc_host_attn_step): per layer two fused residual + norm
        launches, one rotary + cache launch and one attention launch instead of about 45 framework kernels. The
        QKV, output and LM-head projections stay PyTorch matrix products, the FFN is the decode entry point."""
        lib = _lib.lib()
        m = self.model
        cfg = m.config
        heads, hd, t_max = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads, cfg.max_seq_len
        h = m.tok_emb(ids)[:, 0].contiguous()                     # [b, d], updated in place below
        b, d = h.shape
        stream = _lib.stream_ptr(h.device)
        if self._rope_bf16 is None:
            a0 = m.blocks[0].attn
            self._rope_bf16 = (a0.rope_cos.to(h.dtype).contiguous(), a0.rope_sin.to(h.dtype).contiguous())
        cos, sin = self._rope_bf16
        y = torch.empty_like(h)
        q = torch.empty(b, heads * hd, device=h.device, dtype=h.dtype)
        att = torch.empty_like(q)
        ffn_mode = "dense_baseline" if m.ffn_type == "dense" else self.mode
        delta = None
        with torch.cuda.device(h.device):
            for i, blk in enumerate(m.blocks):
                _lib.check(lib.moc_host_rmsnorm(b, d, h.data_ptr(), _lib.ptr(delta), blk.attn_norm.weight.data_ptr(),
                                                y.data_ptr(), blk.attn_norm.eps, stream), "moc_host_rmsnorm")
                qkv = blk.attn.qkv_proj(y)                        # [b, 3 d] = [b, 3, heads, hd]
                _lib.check(lib.moc_host_rope_cache(b, heads, hd, t_max, qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                                   pos.data_ptr(), q.data_ptr(), self.cache_k[i].data_ptr(),
                                                   self.cache_v[i].data_ptr(), stream), "moc_host_rope_cache")
                _lib.check(lib.moc_host_attn_step(b, heads, hd, t_max, q.data_ptr(), self.cache_k[i].data_ptr(),
                                                  self.cache_v[i].data_ptr(), pos.data_ptr(), att.data_ptr(), stream),
                           "moc_host_attn_step")
                o = blk.attn.out_proj(att)
                _lib.check(lib.moc_host_rmsnorm(b, d, h.data_ptr(), o.data_ptr(), blk.ffn_norm.weight.data_ptr(),
                                                y.data_ptr(), blk.ffn_norm.eps, stream), "moc_host_rmsnorm")
                delta = self.ffn[i](y, mode=ffn_mode)
            _lib.check(lib.moc_host_rmsnorm(b, d, h.data_ptr(), _lib.ptr(delta), m.norm.weight.data_ptr(), y.data_ptr(),
                                            m.norm.eps, stream), "moc_host_rmsnorm")
        logits = y @ m.tok_emb.weight.t() if m.lm_head is None else m.lm_head(y)
        return logits.argmax(dim=-1)

    @torch.no_grad()
    def generate_graphed(self, prompt_ids, new_tokens: int):
        """Like generate(), with every decode step after the prompt replayed from one CUDA graph: the token ids,
        the position and the output slot live in device tensors that the graph itself advances, so the loop
        makes no host synchronisation."""
        t0 = prompt_ids.shape[1]
        if t0 + new_tokens > self.model.config.max_seq_len:
            raise ValueError("prompt + new tokens exceed max_seq_len")
        dev = prompt_ids.device
        out = torch.zeros(self.batch, new_tokens, dtype=torch.int64, device=dev)
        first = self._forward(prompt_ids, 0).argmax(dim=-1)
        out[:, 0] = first
        ids = first[:, None].clone()
        pos = torch.full((1,), t0, dtype=torch.int64, device=dev)
        slot = torch.ones(1, dtype=torch.int64, device=dev)

        step = self._step_fused if (self.fused_host_step and self._fused_step_supported()) else self._step

        def body():
            nxt = step(ids, pos)
            out.index_copy_(1, slot, nxt[:, None])
            ids.copy_(nxt[:, None])
            pos.add_(1)
            slot.add_(1)

        if new_tokens > 1:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                # one eager step to warm every lazily created resource up, then rewind and capture
                body()
                pos.fill_(t0)
                slot.fill_(1)
                ids.copy_(first[:, None])
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    body()
                pos.fill_(t0)
                slot.fill_(1)
                ids.copy_(first[:, None])
                for _ in range(new_tokens - 1):
                    graph.replay()
            torch.cuda.current_stream().wait_stream(stream)
            self._graph = graph
        return out

    @torch.no_grad()
    def generate(self, prompt_ids, new_tokens: int):
        """prompt_ids: [batch, T0] int64. Returns [batch, new_tokens] greedy continuations."""
        t0 = prompt_ids.shape[1]
        if t0 + new_tokens > self.model.config.max_seq_len:
            raise ValueError("prompt + new tokens exceed max_seq_len")
        out = []
        nxt = self._forward(prompt_ids, 0).argmax(dim=-1)
        out.append(nxt)
        for step in range(1, new_tokens):
            nxt = self._forward(nxt[:, None], t0 + step - 1).argmax(dim=-1)
            out.append(nxt)
        return torch.stack(out, dim=1)


def synthetic_batch(cfg: HostConfig, batch: int, seq_len: int, pad_fraction: float = 0.1, seed: int = 0,
                    device="cpu"):
    """Token ids uniform over the vocabulary with the trailing `pad_fraction` of every row labelled -100 (the
    label convention of moc/data.py:156-169 on synthetic ids; the model does the causal shift itself)."""
    gen = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab_size, (batch, seq_len), generator=gen)
    labels = ids.clone()
    n_pad = int(round(seq_len * pad_fraction))
    if n_pad:
        labels[:, seq_len - n_pad:] = -100
    return ids.to(device), labels.to(device)


def replace(cfg: HostConfig, **changes) -> HostConfig:
    return dataclasses.replace(cfg, **changes)
