"""Reference arm of bench.py: the UNMODIFIED reference library on the same model and step.

Everything MoE here is the reference's own code, imported from ``baseline/_ref``
(``pip install --target`` of the reference tree) through its public API
(``megablocks.layers.arguments.Arguments`` + ``megablocks.layers.dmoe.dMoE``), on its
stock ``mlp_impl='grouped'`` path.  Two packages the reference imports cannot be
installed offline; ``baseline/shims`` provides import-level stand-ins for them
(``grouped_gemm``: the package's default per-expert cuBLAS loop; ``stk``: container
and decorators only).  The surrounding GPT-2 backbone, data-parallel all-reduce and
mixed-precision Adam are plain PyTorch written here, standing in for the Megatron-LM
fork the reference's scripts use (exp/dmoe/dmoe_125m_8gpu.sh of the reference): bf16
parameters, fp32 main parameters, Adam, clip-grad 1.0, local (non-overlapped) DDP, and the
cosine schedule with 1 % warm-up of those scripts.  Nothing from ``megablocks_b200`` is imported
on this path.
"""

import math
import os
import sys
from functools import partial

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference():
    """Put the installed reference (and the two shims) first on sys.path and import it."""
    ref = os.path.join(HERE, '_ref')
    if not os.path.isdir(os.path.join(ref, 'megablocks')):
        raise ImportError('baseline/_ref/megablocks is missing: the reference is not installed')
    for path in (os.path.join(HERE, 'shims'), ref):
        if path not in sys.path:
            sys.path.insert(0, path)
    import megablocks  # noqa: F401
    from megablocks.layers import dmoe, moe
    from megablocks.layers.arguments import Arguments
    return Arguments, dmoe, moe


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class RefAttention(nn.Module):
    """Multi-head (GPT-2) or grouped-query attention with rotary positions (Mixtral flavour)."""

    def __init__(self, hidden, heads, layers, device, dtype, kv_heads=None, bias=True):
        super().__init__()
        self.heads, self.kv_heads = heads, kv_heads or heads
        self.head_dim = hidden // heads
        self.qkv = nn.Linear(hidden, (heads + 2 * self.kv_heads) * self.head_dim, bias=bias, device=device, dtype=dtype)
        self.proj = nn.Linear(hidden, hidden, bias=bias, device=device, dtype=dtype)
        nn.init.normal_(self.qkv.weight, std=0.02)
        nn.init.normal_(self.proj.weight, std=0.02 / math.sqrt(2.0 * layers))
        if bias:
            nn.init.zeros_(self.qkv.bias)
            nn.init.zeros_(self.proj.bias)

    def forward(self, x, rope=None):
        b, s, h = x.shape
        q_dim, kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        q, k, v = self.qkv(x).split([q_dim, kv_dim, kv_dim], dim=-1)
        q = q.view(b, s, self.heads, self.head_dim).transpose(1, 2)
        k = k.view(b, s, self.kv_heads, self.head_dim).transpose(1, 2)
        v = v.view(b, s, self.kv_heads, self.head_dim).transpose(1, 2)
        if rope is not None:
            q, k = _rope(q, *rope), _rope(k, *rope)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv_heads != self.heads)
        return self.proj(out.transpose(1, 2).reshape(b, s, h))


class RefBlock(nn.Module):

    def __init__(self, cfg, moe_args, dmoe_mod, device, dtype):
        super().__init__()
        mixtral = cfg.get('flavour', 'gpt2') == 'mixtral'
        norm = (lambda n: nn.RMSNorm(n, eps=1e-5, device=device, dtype=dtype)) if mixtral else \
            (lambda n: nn.LayerNorm(n, device=device, dtype=dtype))
        self.ln1 = norm(cfg['hidden'])
        self.attn = RefAttention(cfg['hidden'], cfg['heads'], cfg['layers'], device, dtype,
                                 kv_heads=cfg.get('kv_heads'), bias=not mixtral)
        self.ln2 = norm(cfg['hidden'])
        self.moe = dmoe_mod.dMoE(moe_args)

    def forward(self, x, rope=None):
        x = x + self.attn(self.ln1(x), rope)
        return x + self.moe(self.ln2(x))


class RefGPT(nn.Module):

    def __init__(self, cfg, device, ep_group=None, memory_optimized_mlp=False, recompute=False):
        """``cfg``: hidden, ffn, layers, heads, seq, vocab, experts, top_k and optionally ``flavour``
        ('gpt2' | 'mixtral': RMSNorm, rotary positions, ``kv_heads`` grouped-query attention, SwiGLU
        experts, untied LM head) and ``rope_theta``."""
        super().__init__()
        Arguments, dmoe_mod, self.moe_mod = import_reference()
        dtype = torch.bfloat16
        self.cfg, self.recompute = cfg, recompute
        self.mixtral = cfg.get('flavour', 'gpt2') == 'mixtral'
        self.moe_args = Arguments(
            hidden_size=cfg['hidden'], ffn_hidden_size=cfg['ffn'], num_layers=cfg['layers'], bias=not self.mixtral,
            return_bias=False, activation_fn=F.silu if self.mixtral else partial(F.gelu, approximate='tanh'),
            moe_num_experts=cfg['experts'], moe_top_k=cfg['top_k'], moe_loss_weight=0.1, moe_lbl_in_fp32=True,
            moe_normalize_expert_weights=1 if self.mixtral else None,
            moe_expert_model_parallelism=ep_group is not None, expert_parallel_group=ep_group,
            memory_optimized_mlp=memory_optimized_mlp, mlp_type='glu' if self.mixtral else 'mlp', mlp_impl='grouped',
            fp16=False, bf16=True, device=device,
            init_method=partial(nn.init.normal_, mean=0.0, std=0.02),
            output_layer_init_method=partial(nn.init.normal_, mean=0.0, std=0.02 / math.sqrt(2.0 * cfg['layers'])))
        self.wte = nn.Embedding(cfg['vocab'], cfg['hidden'], device=device, dtype=dtype)
        nn.init.normal_(self.wte.weight, std=0.02)
        self.wpe = self.lm_head = None
        if self.mixtral:
            self.lm_head = nn.Linear(cfg['hidden'], cfg['vocab'], bias=False, device=device, dtype=dtype)
            nn.init.normal_(self.lm_head.weight, std=0.02)
        else:
            self.wpe = nn.Embedding(cfg['seq'], cfg['hidden'], device=device, dtype=dtype)
            nn.init.normal_(self.wpe.weight, std=0.02)
        self.blocks = nn.ModuleList(
            [RefBlock(cfg, self.moe_args, dmoe_mod, device, dtype) for _ in range(cfg['layers'])])
        self.ln_f = nn.RMSNorm(cfg['hidden'], eps=1e-5, device=device, dtype=dtype) if self.mixtral else \
            nn.LayerNorm(cfg['hidden'], device=device, dtype=dtype)
        self._rope = None

    def _rope_tables(self, seq, device):
        if self._rope is None or self._rope[0].shape[0] < seq:
            head_dim = self.cfg['hidden'] // self.cfg['heads']
            inv = 1.0 / (self.cfg.get('rope_theta', 1e6)**(torch.arange(0, head_dim, 2, device=device).float() / head_dim))
            ang = torch.outer(torch.arange(seq, device=device).float(), inv)
            self._rope = (ang.cos(), ang.sin())
        return self._rope[0][:seq], self._rope[1][:seq]

    def loss(self, tokens, targets):
        b, s = tokens.shape
        x = self.wte(tokens)
        rope = None
        if self.mixtral:
            rope = self._rope_tables(s, tokens.device)
        else:
            x = x + self.wpe(torch.arange(s, device=tokens.device))
        for block in self.blocks:
            if self.recompute and self.training:
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(block, x, rope, use_reentrant=False)
            else:
                x = block(x, rope)
        logits = F.linear(self.ln_f(x), self.lm_head.weight if self.mixtral else self.wte.weight)
        lm = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1))
        total = lm + self.moe_mod.batched_load_balancing_loss(self.moe_args)
        self.moe_mod.clear_load_balancing_loss()
        return total, lm.detach()


def cosine_lr(step, total_steps, peak, floor, warmup_fraction=0.01):
    """Linear warm-up, then cosine decay (--lr-decay-style cosine --lr-warmup-fraction 0.01)."""
    warm = max(1, int(total_steps * warmup_fraction))
    if step < warm:
        return peak * (step + 1) / warm
    frac = min(1.0, (step - warm) / max(1, total_steps - warm))
    return floor + 0.5 * (peak - floor) * (1.0 + math.cos(math.pi * frac))


class ExposedCommTimer:
    """Times the all-to-alls the reference issues, as seen from the compute stream.

    ``torch.distributed.all_to_all_single`` is wrapped (the reference itself is untouched): a
    blocking call is bracketed by two CUDA events, an ``async_op`` call returns a handle whose
    ``wait()`` is bracketed instead - the part of the exchange the compute stream actually waits for.
    """

    def __init__(self):
        self.enabled = False
        self.pairs = []
        self._orig = dist.all_to_all_single
        timer = self

        class Handle:
            def __init__(self, work):
                self.work = work

            def wait(self, *args, **kwargs):
                if not timer.enabled:
                    return self.work.wait(*args, **kwargs)
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                out = self.work.wait(*args, **kwargs)
                end.record()
                timer.pairs.append((start, end))
                return out

            def __getattr__(self, name):
                return getattr(self.work, name)

        def wrapped(*args, **kwargs):
            if not timer.enabled:
                return timer._orig(*args, **kwargs)
            if kwargs.get('async_op'):
                return Handle(timer._orig(*args, **kwargs))
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = timer._orig(*args, **kwargs)
            end.record()
            timer.pairs.append((start, end))
            return out

        dist.all_to_all_single = wrapped

    def reset(self):
        self.pairs = []

    def total_ms(self):
        torch.cuda.synchronize()
        return float(sum(s.elapsed_time(e) for s, e in self.pairs))


class RefTrainer:
    """bf16 model parameters, fp32 main parameters, Adam, clip-grad 1.0, local DDP."""

    def __init__(self, model, lr=6e-4, min_lr=6e-5, total_steps=20000, world=1, group=None):
        self.model, self.world, self.group = model, world, group
        self.lr, self.min_lr, self.total_steps, self.step_count = lr, min_lr, total_steps, 0
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.dense = [p for p in self.params if not getattr(p, 'expert_model_parallel', False)]
        self.main = [p.detach().clone().float().requires_grad_(True) for p in self.params]
        self.opt = torch.optim.Adam(self.main, lr=lr, betas=(0.9, 0.95), eps=1e-8, fused=True)
        self.device = self.params[0].device

    def step(self, tokens, targets):
        self.model.train()
        for p in self.params:
            p.grad = None
        total, lm = self.model.loss(tokens, targets)
        total.backward()
        if self.world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in self.dense])
            dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group)
            off = 0
            for p in self.dense:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p))
                off += p.numel()
        for m, p in zip(self.main, self.params):
            m.grad = p.grad.float()
        sq = torch.stack([g.grad.square().sum() * (1.0 if getattr(p, 'expert_model_parallel', False) or
                                                    self.world == 1 else 1.0 / self.world)
                          for g, p in zip(self.main, self.params)]).sum()
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        coeff = torch.clamp(1.0 / (sq.sqrt() + 1e-6), max=1.0)
        torch._foreach_mul_([m.grad for m in self.main], coeff)
        for group in self.opt.param_groups:
            group['lr'] = cosine_lr(self.step_count, self.total_steps, self.lr, self.min_lr)
        self.step_count += 1
        self.opt.step()
        with torch.no_grad():
            torch._foreach_copy_(self.params, self.main)
        return lm

    def step_from_host(self, batch):
        dev = batch.to(self.device, non_blocking=True)
        return float(self.step(dev[:, :-1], dev[:, 1:]).item())

    def run_from_host(self, batches):
        """The same training loop as the library arm's ``Trainer.run_from_host``: one step per pinned
        host batch, every loss copied back to pinned memory and read after the next step is queued."""
        losses, pending = [], None
        ring = [torch.empty(1, dtype=torch.float32, pin_memory=True) for _ in range(2)]
        events = [torch.cuda.Event() for _ in range(2)]
        for i, batch in enumerate(batches):
            dev = batch.to(self.device, non_blocking=True)
            loss = self.step(dev[:, :-1], dev[:, 1:])
            slot = i & 1
            ring[slot].copy_(loss.detach().float().reshape(1), non_blocking=True)
            events[slot].record()
            if pending is not None:
                events[pending].synchronize()
                losses.append(float(ring[pending][0]))
            pending = slot
        if pending is not None:
            events[pending].synchronize()
            losses.append(float(ring[pending][0]))
        return losses
