"""Stand-alone trainer for the dMoE transformer family.

Takes the place of the Megatron-LM fork the reference's experiment scripts
launch (exp/dmoe/dmoe_125m_8gpu.sh:159-167): bf16 parameters with fp32 master
weights, Adam, gradient clipping, cosine schedule, expert parallelism over the
whole job with the non-expert parameters data-parallel (gradient reduction
overlapped with backward, optionally ZeRO-1 sharded), synthetic or
caller-supplied token batches.

    trainer = Trainer(model, TrainerConfig(lr=6e-4), dp_group=group)
    loss = trainer.step(tokens, targets)            # device tensors
    loss = trainer.step_from_host(batch_cpu)        # pinned host tokens -> float

One process drives one GPU; ``torch.distributed`` (NCCL) connects them.
"""

import dataclasses
import time
from typing import Optional

import torch
import torch.distributed as dist

from megablocks_b200.layers import mpu
from megablocks_b200.optim import FusedAdam, clip_coefficient, cosine_lr
from megablocks_b200.parallel.dp import FlatBuffer, GradReducer


@dataclasses.dataclass
class TrainerConfig:
    lr: float = 6e-4
    min_lr: float = 6e-5
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    total_steps: int = 20000
    warmup_fraction: float = 0.01
    zero1: bool = False              # shard optimizer state of the replicated parameters
    bucket_mb: int = 32
    schedule: bool = True
    # Run the (bandwidth-bound) Adam update of the expert weights on a side stream, layer by layer,
    # while the next step's forward already runs; every MoE layer waits for its own weights only.
    # CUDA only.  Off by default: measured on B200 with the 125M dMoE it changes nothing, because
    # the forward's persistent GEMM CTAs occupy whole SMs and the update runs between them anyway.
    overlap_expert_update: bool = False


class Trainer:

    def __init__(self, model: torch.nn.Module, cfg: TrainerConfig, dp_group: Optional[dist.ProcessGroup] = None):
        self.model, self.cfg, self.dp_group = model, cfg, dp_group
        self.world = dist.get_world_size(dp_group) if (dist.is_initialized() and dp_group is not None) else 1
        params = [p for p in model.parameters() if p.requires_grad]
        # "Expert" parameters are the ones no other rank holds a replica of: the expert-parallel shards,
        # or, in a single process, everything a MoE layer owns (they get their own optimizer group so
        # that its update can be deferred layer by layer).
        if self.world > 1:
            expert_ids = {id(p) for p in params if mpu.param_is_expert_model_parallel(p)}
        else:
            from megablocks_b200.layers.moe import MoE
            expert_ids = {id(p) for m in model.modules() if isinstance(m, MoE) for p in m.parameters()}
        self.expert_params = [p for p in params if id(p) in expert_ids]
        self.dense_params = [p for p in params if id(p) not in expert_ids]
        self.device = params[0].device
        self._update_stream = None
        self._update_groups = []     # (module, first tensor, one past the last tensor) in forward order
        self._pending_updates = {}   # module -> event recorded after its expert weights were updated
        if self.expert_params:
            self._plan_expert_update_groups(cfg.overlap_expert_update and self.device.type == 'cuda')
        self.flat = self.reducer = None
        kw = dict(lr=cfg.lr, betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay)
        if self.world > 1:
            self.flat = FlatBuffer(self.dense_params, granule=self.world * 8)
            self.reducer = GradReducer(self.flat, dp_group, cfg.bucket_mb << 20, shard=cfg.zero1)
        if self.world > 1 and cfg.zero1:
            # One optimizer "tensor" per owned bucket slice; disjoint across ranks.
            self._shard_params, self._shard_grads = [], []
            for bi in range(len(self.reducer.buckets)):
                lo, hi = self.reducer.shard_range(bi)
                self._shard_params.append(self.flat.param[lo:hi])
                self._shard_grads.append(self.flat.grad[lo:hi])
            self.dense_opt = FusedAdam(self._shard_params, **kw)
        else:
            # Replicated tensors: count their norm once across the group.
            self.dense_opt = FusedAdam(self.dense_params, norm_weights=[1.0 / self.world] * len(self.dense_params),
                                       **kw)
        self.expert_opt = FusedAdam(self.expert_params, **kw)
        self._sqnorm = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.step_count = 0
        self.last_grad_norm = None
        self._h2d = None

    # -- deferred expert update ------------------------------------------------------
    def _plan_expert_update_groups(self, deferred: bool) -> None:
        """Order the expert weights by the MoE layer that owns them; with ``deferred`` also hook those
        layers so each waits for its own side-stream update."""
        from megablocks_b200.layers.moe import MoE
        is_expert = {id(p) for p in self.expert_params}
        ordered, groups, seen = [], [], set()
        for module in self.model.modules():
            if not isinstance(module, MoE):
                continue
            own = [p for p in module.parameters() if id(p) in is_expert and id(p) not in seen and p.requires_grad]
            if own:
                seen.update(id(p) for p in own)
                groups.append((module, len(ordered), len(ordered) + len(own)))
                ordered += own
        rest = [p for p in self.expert_params if id(p) not in seen]
        if rest:   # expert weights outside any MoE layer: needed from the very start of the forward pass
            groups = [(self.model, 0, len(rest))] + [(m, lo + len(rest), hi + len(rest)) for (m, lo, hi) in groups]
            ordered = rest + ordered
        self.expert_params = ordered
        self._update_groups = groups
        if deferred:
            self._update_stream = torch.cuda.Stream(device=self.device)
            for module, _, _ in groups:
                module.register_forward_pre_hook(self._wait_for_update)

    def _wait_for_update(self, module, _inputs):
        event = self._pending_updates.pop(module, None)
        if event is not None:
            torch.cuda.current_stream().wait_event(event)

    def flush(self) -> None:
        """Make the current stream wait for every deferred expert update (before reading the weights
        outside a forward pass, saving a checkpoint, or closing a timed region)."""
        if self._update_stream is not None:
            torch.cuda.current_stream().wait_stream(self._update_stream)
            self._pending_updates.clear()

    def _step_experts(self, coeff: torch.Tensor) -> None:
        if self._update_stream is None:
            self.expert_opt.step(coeff)
            return
        grads = self.expert_opt.grads()
        side = self._update_stream
        self.expert_opt.begin_step(grads)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for module, lo, hi in self._update_groups:
                self.expert_opt.step_range(lo, hi, coeff, grads)
                event = torch.cuda.Event()
                event.record(side)
                self._pending_updates[module] = event
        # The gradients (dropped at the start of the next step) and the coefficient are still being
        # read on the side stream: keep the allocator from recycling them too early.
        for g in grads:
            g.record_stream(side)
        coeff.record_stream(side)

    # -- one optimisation step ---------------------------------------------------------
    def _zero_grad(self):
        if self.flat is not None:
            self.flat.zero_grad()
        else:
            for p in self.dense_params:
                p.grad = None
        for p in self.expert_params:
            p.grad = None

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Forward, backward, gradient reduction, clipping and the optimizer update.

        Returns the language-model loss as a device scalar (no host sync).
        """
        cfg = self.cfg
        self.model.train()
        self._zero_grad()
        total, lm = self.model.loss(tokens, targets)
        total.backward()
        if self.reducer is not None:
            self.reducer.finish()
        lr = cosine_lr(self.step_count, cfg.total_steps, cfg.lr, cfg.min_lr, cfg.warmup_fraction) if cfg.schedule \
            else cfg.lr
        self.dense_opt.lr = self.expert_opt.lr = lr

        dense_grads = self._shard_grads if (self.world > 1 and cfg.zero1) else None
        self.flush()   # a layer that did not run this step may still have an update in flight
        self._sqnorm.zero_()
        self.dense_opt.add_sqnorm(self._sqnorm, dense_grads)
        self.expert_opt.add_sqnorm(self._sqnorm)
        if self.world > 1:
            dist.all_reduce(self._sqnorm, group=self.dp_group)
        coeff = clip_coefficient(self._sqnorm, cfg.max_grad_norm)
        self.last_grad_norm = coeff[1:2]
        self.dense_opt.step(coeff[0:1], dense_grads)
        self._step_experts(coeff[0:1])
        if self.world > 1 and cfg.zero1:
            self.reducer.gather_params()
        self.step_count += 1
        return lm

    # -- end-to-end step from host memory ---------------------------------------------
    def step_from_host(self, batch: torch.Tensor) -> float:
        """``batch`` is a pinned int64 host tensor ``[micro_batch, seq + 1]``.

        Copies it to the device, trains one step on (batch[:, :-1] -> batch[:, 1:])
        and reads the loss back to the host.
        """
        dev = batch.to(self.device, non_blocking=True)
        loss = self.step(dev[:, :-1], dev[:, 1:])
        return float(loss.item())

    def state_dict(self):
        self.flush()
        return {'model': self.model.state_dict(), 'dense_opt': self.dense_opt.state_dict(),
                'expert_opt': self.expert_opt.state_dict(), 'step': self.step_count}

    def load_state_dict(self, state):
        self.flush()
        self.model.load_state_dict(state['model'])
        self.dense_opt.load_state_dict(state['dense_opt'])
        self.expert_opt.load_state_dict(state['expert_opt'])
        self.step_count = int(state['step'])


def synthetic_batch(micro_batch: int, seq_len: int, vocab_size: int, generator: Optional[torch.Generator] = None,
                    pin: bool = True) -> torch.Tensor:
    """Uniform-random token ids ``[micro_batch, seq_len + 1]`` in (pinned) host memory."""
    batch = torch.randint(0, vocab_size, (micro_batch, seq_len + 1), generator=generator, dtype=torch.int64)
    return batch.pin_memory() if pin and torch.cuda.is_available() else batch


# ---------------------------------------------------------------------------
# Command line: python -m megablocks_b200.train --preset dmoe-125m ...
# ---------------------------------------------------------------------------
def main(argv=None):
    import argparse
    import os

    from megablocks_b200 import checkpoint
    from megablocks_b200.models.transformer import MoETransformer, PRESETS, preset
    from megablocks_b200.utils import status
    from megablocks_b200.utils.health import Heartbeat
    from megablocks_b200.utils.metrics import JsonlLogger, expert_load_stats, nvtx_range

    ap = argparse.ArgumentParser(description='Train a dMoE / MoE transformer on synthetic tokens.')
    ap.add_argument('--preset', choices=sorted(PRESETS), default='dmoe-125m')
    ap.add_argument('--micro-batch', type=int, default=32)
    ap.add_argument('--steps', type=int, default=100)
    ap.add_argument('--experts', type=int, default=None)
    ap.add_argument('--top-k', type=int, default=None)
    ap.add_argument('--loss-weight', type=float, default=0.1)
    ap.add_argument('--capacity-factor', type=int, default=None, help='token-dropping MoE with this capacity factor')
    ap.add_argument('--mlp-impl', choices=['grouped', 'sparse'], default='grouped')
    ap.add_argument('--lr', type=float, default=6e-4)
    ap.add_argument('--min-lr', type=float, default=6e-5)
    ap.add_argument('--zero1', action='store_true', help='shard the optimizer state of the replicated parameters')
    ap.add_argument('--recompute', action='store_true', help='activation checkpointing of every block')
    ap.add_argument('--defer-expert-update', action='store_true',
                    help='run the expert Adam update on a side stream, layer by layer, under the next forward')
    ap.add_argument('--ep-comm', choices=['auto', 'fused', 'nccl'], default='auto')
    ap.add_argument('--log', type=str, default=None, help='JSONL metrics file')
    ap.add_argument('--log-interval', type=int, default=10)
    ap.add_argument('--save', type=str, default=None, help='checkpoint directory')
    ap.add_argument('--save-interval', type=int, default=0)
    ap.add_argument('--load', type=str, default=None)
    ap.add_argument('--seed', type=int, default=1234)
    args = ap.parse_args(argv)

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    use_cuda = torch.cuda.is_available()
    device = torch.device('cuda', local) if use_cuda else torch.device('cpu')
    if use_cuda:
        torch.cuda.set_device(local)
    group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29500')
        dist.init_process_group('nccl' if use_cuda else 'gloo', rank=rank, world_size=world)
        group = dist.group.WORLD

    torch.manual_seed(args.seed)
    overrides = dict(device=device, expert_parallel_group=group, mlp_impl=args.mlp_impl,
                     moe_loss_weight=args.loss_weight, activation_checkpointing=args.recompute,
                     ep_fused_comm={'auto': None, 'fused': True, 'nccl': False}[args.ep_comm],
                     dtype=torch.bfloat16 if use_cuda else torch.float32)
    if args.experts is not None:
        overrides['moe_num_experts'] = args.experts
    if args.top_k is not None:
        overrides['moe_top_k'] = args.top_k
    if args.capacity_factor is not None:
        overrides.update(dropless=False, moe_capacity_factor=args.capacity_factor)
    cfg = preset(args.preset, **overrides)
    model = MoETransformer(cfg)
    trainer = Trainer(model, TrainerConfig(lr=args.lr, min_lr=args.min_lr, total_steps=args.steps, zero1=args.zero1,
                                           overlap_expert_update=args.defer_expert_update),
                      dp_group=group)
    if args.load:
        state = checkpoint.load(args.load, rank, world, map_location=device)
        model.load_state_dict(state['model'])
        if 'dense_opt' in state:
            trainer.load_state_dict(state)
    logger = JsonlLogger(args.log, rank)
    heartbeat = Heartbeat(timeout_s=60.0) if world > 1 else None
    gen = torch.Generator().manual_seed(args.seed + rank)
    tokens_per_step = world * args.micro_batch * cfg.max_seq_len
    t_last, loss = time.time(), None
    for step in range(trainer.step_count, args.steps):
        if heartbeat is not None:
            heartbeat.check()
        batch = synthetic_batch(args.micro_batch, cfg.max_seq_len, cfg.vocab_size, gen)
        with nvtx_range('train_step'):
            dev = batch.to(device, non_blocking=True)
            loss = trainer.step(dev[:, :-1], dev[:, 1:])
        if heartbeat is not None:
            heartbeat.beat()
        if (step + 1) % args.log_interval == 0 or step + 1 == args.steps:
            value = float(loss)                      # the only host sync of the interval
            if use_cuda:
                status.check()
            now = time.time()
            rate = tokens_per_step * args.log_interval / max(now - t_last, 1e-9)
            t_last = now
            logger.log(step=step + 1, loss=value, grad_norm=trainer.last_grad_norm, tokens_per_s=rate,
                       lr=trainer.dense_opt.lr)
            if rank == 0:
                print(f'step {step + 1:6d}  loss {value:8.4f}  grad-norm {float(trainer.last_grad_norm):7.3f}  '
                      f'{rate:12.0f} tokens/s', flush=True)
        if args.save and args.save_interval and (step + 1) % args.save_interval == 0:
            checkpoint.save(args.save, trainer.state_dict(), rank, world, cfg.moe_num_experts, step + 1)
    if args.save:
        checkpoint.save(args.save, trainer.state_dict(), rank, world, cfg.moe_num_experts, trainer.step_count)
    logger.close()
    if world > 1:
        dist.destroy_process_group()
    return loss


if __name__ == '__main__':
    main()
