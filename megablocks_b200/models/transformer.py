"""Decoder-only transformers whose feed-forward blocks are dMoE / MoE layers.

The reference ships no model code: its experiment scripts train GPT-2 style
models through a Megatron-LM fork that replaces every FFN with a dMoE layer
(exp/dmoe/dmoe_125m_8gpu.sh:53-72,143-148).  This module provides that model
family natively so the library can be trained and benchmarked stand-alone:

* ``gpt2`` flavour: LayerNorm, learned positions, GELU experts, tied LM head;
* ``mixtral`` flavour: RMSNorm, rotary positions, grouped-query attention,
  SwiGLU experts (``mlp_type='glu'``), untied LM head.

Attention uses the library fused attention (``scaled_dot_product_attention``);
everything MoE runs this library's kernels.  Inputs are ``[batch, seq]`` token ids.
"""

import dataclasses
import math
from functools import partial
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from megablocks_b200.layers.arguments import Arguments
from megablocks_b200.layers.dmoe import dMoE
from megablocks_b200.layers.moe import MoE, batched_load_balancing_loss, clear_load_balancing_loss
from megablocks_b200.layers.router import batched_router_zloss, clear_router_zloss
from megablocks_b200.ops import fused


@dataclasses.dataclass
class TransformerConfig:
    flavour: str = 'gpt2'               # 'gpt2' | 'mixtral'
    vocab_size: int = 51200
    max_seq_len: int = 1024
    num_layers: int = 12
    hidden_size: int = 768
    num_heads: int = 12
    num_kv_heads: Optional[int] = None  # grouped-query attention when < num_heads
    ffn_hidden_size: int = 3072
    moe_num_experts: int = 64
    moe_top_k: int = 1
    moe_loss_weight: float = 0.1
    moe_zloss_weight: float = 0.0
    moe_capacity_factor: int = 1
    dropless: bool = True
    mlp_impl: str = 'grouped'
    memory_optimized_mlp: bool = True
    rope_theta: float = 10000.0
    init_std: float = 0.02
    activation_checkpointing: bool = False
    dtype: torch.dtype = torch.bfloat16
    device: Optional[torch.device] = None
    # expert parallelism
    expert_parallel_group: Optional[object] = None
    ep_fused_comm: Optional[bool] = None
    ep_inflight_microbatches: int = 1
    # pipeline parallelism: this process builds stage `pipeline_stage` of `pipeline_stages`
    pipeline_stages: int = 1
    pipeline_stage: int = 0

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads or self.num_heads

    def moe_arguments(self) -> Arguments:
        glu = self.flavour == 'mixtral'
        return Arguments(
            hidden_size=self.hidden_size,
            ffn_hidden_size=self.ffn_hidden_size,
            num_layers=self.num_layers,
            bias=not glu,
            return_bias=True,      # the bias add rides in the next norm kernel (Block.forward)
            activation_fn=F.silu if glu else partial(F.gelu, approximate='tanh'),
            moe_num_experts=self.moe_num_experts,
            moe_top_k=self.moe_top_k,
            moe_capacity_factor=self.moe_capacity_factor,
            moe_loss_weight=self.moe_loss_weight,
            moe_zloss_weight=self.moe_zloss_weight,
            moe_lbl_in_fp32=True,
            moe_normalize_expert_weights=1 if glu else None,
            moe_expert_model_parallelism=self.expert_parallel_group is not None,
            expert_parallel_group=self.expert_parallel_group,
            memory_optimized_mlp=self.memory_optimized_mlp,
            mlp_type='glu' if glu else 'mlp',
            mlp_impl=self.mlp_impl,
            fp16=self.dtype == torch.float16,
            bf16=self.dtype == torch.bfloat16,
            device=self.device if self.device is not None else torch.device('cpu'),
            init_method=partial(nn.init.normal_, mean=0.0, std=self.init_std),
            output_layer_init_method=partial(nn.init.normal_, mean=0.0,
                                             std=self.init_std / math.sqrt(2.0 * self.num_layers)),
            ep_fused_comm=self.ep_fused_comm,
            ep_inflight_microbatches=self.ep_inflight_microbatches,
            pipeline_model_parallel_size=self.pipeline_stages,
        )


# Named configurations: the dMoE family trained by the reference's experiment
# scripts (exp/dmoe/*.sh: 64 experts, top-1, ffn = 4 x hidden, seq 1024) and a
# Mixtral-8x7B-shaped model.
PRESETS = {
    'dmoe-46m': dict(num_layers=6, hidden_size=512, num_heads=8, ffn_hidden_size=2048),
    'dmoe-125m': dict(num_layers=12, hidden_size=768, num_heads=12, ffn_hidden_size=3072),
    'dmoe-356m': dict(num_layers=24, hidden_size=1024, num_heads=16, ffn_hidden_size=4096),
    'dmoe-760m': dict(num_layers=24, hidden_size=1536, num_heads=16, ffn_hidden_size=6144),
    'dmoe-1315m': dict(num_layers=24, hidden_size=2048, num_heads=16, ffn_hidden_size=8192),
    'mixtral-8x7b': dict(flavour='mixtral', vocab_size=32000, max_seq_len=4096, num_layers=32, hidden_size=4096,
                         num_heads=32, num_kv_heads=8, ffn_hidden_size=14336, moe_num_experts=8, moe_top_k=2,
                         rope_theta=1e6),
    'tiny': dict(vocab_size=512, max_seq_len=64, num_layers=2, hidden_size=128, num_heads=4, ffn_hidden_size=256,
                 moe_num_experts=8, moe_top_k=2),
    'tiny-mixtral': dict(flavour='mixtral', vocab_size=512, max_seq_len=64, num_layers=2, hidden_size=128,
                         num_heads=4, num_kv_heads=2, ffn_hidden_size=256, moe_num_experts=4, moe_top_k=2),
}


def preset(name: str, **overrides) -> TransformerConfig:
    cfg = dict(PRESETS[name])
    cfg.update(overrides)
    return TransformerConfig(**cfg)


RMSNorm = fused.RMSNorm


def _rope_tables(seq_len: int, head_dim: int, theta: float, device):
    inv = 1.0 / (theta**(torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


class Attention(nn.Module):

    def __init__(self, cfg: TransformerConfig):
        super().__init__()
        self.cfg = cfg
        self.head_dim = cfg.hidden_size // cfg.num_heads
        kw = dict(device=cfg.device, dtype=cfg.dtype)
        bias = cfg.flavour == 'gpt2'
        qkv_out = (cfg.num_heads + 2 * cfg.kv_heads) * self.head_dim
        self.qkv = fused.Linear(cfg.hidden_size, qkv_out, bias=bias, **kw)
        self.proj = fused.Linear(cfg.hidden_size, cfg.hidden_size, bias=bias, **kw)
        nn.init.normal_(self.qkv.weight, std=cfg.init_std)
        nn.init.normal_(self.proj.weight, std=cfg.init_std / math.sqrt(2.0 * cfg.num_layers))
        if bias:
            nn.init.zeros_(self.qkv.bias)
            nn.init.zeros_(self.proj.bias)

    def forward(self, x: torch.Tensor, rope) -> torch.Tensor:
        b, s, _ = x.shape
        cfg = self.cfg
        qkv = self.qkv(x)
        q_dim, kv_dim = cfg.num_heads * self.head_dim, cfg.kv_heads * self.head_dim
        q, k, v = qkv.split([q_dim, kv_dim, kv_dim], dim=-1)
        q = q.view(b, s, cfg.num_heads, self.head_dim)
        k = k.view(b, s, cfg.kv_heads, self.head_dim)
        if rope is not None:     # rotate the [batch, seq, heads, dim] views of the fused projection in one pass each
            q, k = fused.rope(q, *rope), fused.rope(k, *rope)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        v = v.view(b, s, cfg.kv_heads, self.head_dim).transpose(1, 2)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=cfg.kv_heads != cfg.num_heads)
        return self.proj(out.transpose(1, 2).reshape(b, s, -1))


def _add_norm(norm: nn.Module, x: torch.Tensor, delta, delta_bias=None):
    """``(x + delta [+ delta_bias], norm(...))``; ``delta_bias`` is the per-column output bias of the
    layer that produced ``delta``."""
    if hasattr(norm, 'add_forward'):
        return norm.add_forward(x, delta, delta_bias)
    if delta is not None:
        x = x + delta if delta_bias is None else x + delta + delta_bias
    return x, norm(x)


class Block(nn.Module):

    def __init__(self, cfg: TransformerConfig, moe_args: Arguments):
        super().__init__()
        kw = dict(device=cfg.device, dtype=cfg.dtype)
        norm = RMSNorm if cfg.flavour == 'mixtral' else fused.LayerNorm
        self.ln1 = norm(cfg.hidden_size, **kw)
        self.attn = Attention(cfg)
        self.ln2 = norm(cfg.hidden_size, **kw)
        self.moe = (dMoE if cfg.dropless else MoE)(moe_args)

    def forward(self, x: torch.Tensor, delta, delta_bias, rope):
        """The residual stream arrives as ``x + delta + delta_bias`` (``delta`` may be ``None``;
        ``delta_bias`` is the previous MoE layer's output bias, one value per column, or ``None``)
        and leaves the same way, so every residual add rides in the following norm's kernels."""
        x, normed = _add_norm(self.ln1, x, delta, delta_bias)
        x, normed = _add_norm(self.ln2, x, self.attn(normed, rope))
        # The MoE layer is token-wise: it flattens every leading dimension, so the
        # [batch, seq, hidden] activations go in as they are (no transpose copy).
        out = self.moe(normed)
        if isinstance(out, tuple):        # return_bias: (output without the bias, bias vector)
            return x, out[0], out[1]
        return x, out, None


class MoETransformer(nn.Module):
    """Token ids ``[batch, seq]`` -> logits ``[batch, seq, vocab]`` (and the training loss)."""

    def __init__(self, cfg: TransformerConfig):
        super().__init__()
        self.cfg = cfg
        self.moe_args = cfg.moe_arguments()
        kw = dict(device=cfg.device, dtype=cfg.dtype)
        # A pipeline stage owns a contiguous slice of the blocks; the first stage also owns the
        # embeddings, the last one the final norm and the LM head (which is then a matrix of its
        # own: the tied GPT-2 head would need the embedding of another process).
        from megablocks_b200.parallel.pipeline import stage_layers
        if cfg.pipeline_stages > 1 and cfg.num_layers % cfg.pipeline_stages:
            raise ValueError('num_layers must be divisible by pipeline_stages (the load-balancing loss expects '
                             'num_layers / pipeline_stages terms per stage)')
        self.is_first_stage = cfg.pipeline_stage == 0
        self.is_last_stage = cfg.pipeline_stage == cfg.pipeline_stages - 1
        self.wte = self.wpe = self.ln_f = self.lm_head = None
        if self.is_first_stage:
            self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden_size, **kw)
            nn.init.normal_(self.wte.weight, std=cfg.init_std)
            if cfg.flavour == 'gpt2':
                self.wpe = nn.Embedding(cfg.max_seq_len, cfg.hidden_size, **kw)
                nn.init.normal_(self.wpe.weight, std=cfg.init_std)
        layers = stage_layers(cfg.num_layers, cfg.pipeline_stages, cfg.pipeline_stage)
        self.blocks = nn.ModuleList([Block(cfg, self.moe_args) for _ in layers])
        norm = RMSNorm if cfg.flavour == 'mixtral' else fused.LayerNorm
        if self.is_last_stage:
            self.ln_f = norm(cfg.hidden_size, **kw)
            if cfg.flavour == 'mixtral' or not self.is_first_stage:
                self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, **kw)
                nn.init.normal_(self.lm_head.weight, std=cfg.init_std)
        self._rope = None

    def _rope_for(self, seq: int, device):
        if self.cfg.flavour != 'mixtral':
            return None
        if self._rope is None or self._rope[0].shape[0] < seq or self._rope[0].device != device:
            head_dim = self.cfg.hidden_size // self.cfg.num_heads
            self._rope = _rope_tables(max(seq, self.cfg.max_seq_len), head_dim, self.cfg.rope_theta, device)
        return self._rope[0][:seq], self._rope[1][:seq]

    def _embed(self, tokens: torch.Tensor) -> torch.Tensor:
        x = self.wte(tokens)
        if self.wpe is not None:
            x = x + self.wpe(torch.arange(tokens.shape[1], device=tokens.device))
        return x

    def _run_blocks(self, x: torch.Tensor):
        """Residual stream through this process's blocks; returns ``(x, delta, delta_bias)`` with the
        last block's output (and its bias vector, if any) still to be added."""
        rope = self._rope_for(x.shape[1], x.device)
        delta = delta_bias = None
        for block in self.blocks:
            if self.cfg.activation_checkpointing and self.training:
                x, delta, delta_bias = checkpoint(block, x, delta, delta_bias, rope, use_reentrant=False)
            else:
                x, delta, delta_bias = block(x, delta, delta_bias, rope)
        return x, delta, delta_bias

    def hidden_states(self, tokens: torch.Tensor) -> torch.Tensor:
        x, delta, delta_bias = self._run_blocks(self._embed(tokens))
        return _add_norm(self.ln_f, x, delta, delta_bias)[1]

    def _aux_loss(self):
        """This stage's auxiliary losses of the forward pass just run (``None`` when there are none);
        clears the per-step accumulators."""
        aux = None
        if self.training and self.moe_args.moe_loss_weight > 0:
            aux = batched_load_balancing_loss(self.moe_args)
        if self.training and self.moe_args.moe_zloss_weight > 0:
            z = batched_router_zloss(self.moe_args).sum()
            aux = z if aux is None else aux + z
        clear_load_balancing_loss()
        clear_router_zloss()
        return aux

    # -- pipeline stages ---------------------------------------------------------------
    def stage_forward(self, inp: torch.Tensor):
        """One pipeline stage: token ids (first stage) or the previous stage's activations in,
        ``(activations for the next stage, auxiliary loss of this stage or None)`` out.  The last
        stage returns the un-normalised residual stream for :meth:`stage_loss`."""
        x, delta, delta_bias = self._run_blocks(self._embed(inp) if self.is_first_stage else inp)
        if delta is not None:
            x = x + delta if delta_bias is None else x + delta + delta_bias
        return x, self._aux_loss()

    def stage_loss(self, hidden: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Last stage: final norm, LM head and cross entropy."""
        return self._lm_loss(self.ln_f(hidden), targets)

    def _lm_loss(self, hidden: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Language-model head and mean cross entropy (the logits are written once and read once)."""
        weight = self.lm_head.weight if self.lm_head is not None else self.wte.weight
        return fused.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), weight, targets.reshape(-1))

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        weight = self.lm_head.weight if self.lm_head is not None else self.wte.weight
        return F.linear(hidden, weight)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.logits(self.hidden_states(tokens))

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor):
        """Next-token cross entropy plus the MoE auxiliary losses.

        Returns ``(total, lm_loss)``.  Clears the per-step loss accumulators.
        """
        if self.cfg.pipeline_stages > 1:
            raise RuntimeError('a pipeline stage is driven through stage_forward / stage_loss')
        lm = self._lm_loss(self.hidden_states(tokens), targets)
        aux = self._aux_loss()
        total = lm if aux is None else lm + aux
        return total, lm.detach()

    def num_parameters(self, only_active: bool = False) -> int:
        total = 0
        for name, p in self.named_parameters():
            n = p.numel()
            if only_active and '.moe.experts.mlp.' in name:
                n = n * self.cfg.moe_top_k // max(1, p.shape[0] // self.cfg.ffn_hidden_size)
            total += n
        return total
