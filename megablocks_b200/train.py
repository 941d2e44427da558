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
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from megablocks_b200.layers import mpu
from megablocks_b200.optim import Adafactor, DynamicLossScaler, FusedAdam, clip_coefficient, cosine_lr
from megablocks_b200.parallel.dp import FlatBuffer, GradReducer
from megablocks_b200.utils.metrics import nvtx_range


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
    # Data-parallel gradient reduction: 'peer' = this library's kernel over NVLink peer memory,
    # 'nccl' = library collectives, 'auto' = peer on CUDA, nccl otherwise.
    dp_backend: str = 'auto'
    schedule: bool = True
    # Run the (bandwidth-bound) Adam update of the expert weights on a side stream, layer by layer,
    # while the next step's forward already runs; every MoE layer waits for its own weights only.
    # CUDA only.  Off by default: measured on B200 with the 125M dMoE it changes nothing, because
    # the forward's persistent GEMM CTAs occupy whole SMs and the update runs between them anyway.
    overlap_expert_update: bool = False
    # One optimizer step covers `grad_accum_steps` micro-batches: `step` splits its batch along
    # dimension 0, the gradients add up in place and the data-parallel reduction starts during the
    # backward pass of the last micro-batch only (the reference's recipes: global batch 512 on
    # 8 GPUs x micro-batch 32 = 2 micro-batches per step, exp/dmoe/dmoe_125m_8gpu.sh:5-9,63).
    grad_accum_steps: int = 1
    optimizer: str = 'adam'          # 'adam' | 'adafactor' (exp/dmoe/dmoe_760m_8gpu.sh)
    # fp16 parameters train under dynamic loss scaling (None = on exactly when the model is fp16).
    loss_scaling: Optional[bool] = None
    init_loss_scale: float = 2.0**16
    loss_scale_window: int = 1000
    # Record the whole step (forward, backward, norm, clip, both Adam updates) in ONE CUDA graph
    # after `graph_warmup_steps` ordinary steps and replay it from then on.  Possible because no
    # kernel of the step needs a size from the host: group sizes, the clip coefficient, the learning
    # rate and Adam's bias corrections are all read from device memory.  Single process, bf16/fp32,
    # fused Adam, fixed batch shape; anything else keeps running step by step.
    cuda_graph: bool = False
    graph_warmup_steps: int = 3
    # Take the squared norm of the expert weight gradients in the epilogue of the GEMMs that
    # produce them instead of reading the gradients back for it (one optimizer step per backward
    # pass only: no gradient accumulation, no pipeline).
    fuse_grad_norm: bool = True


class Trainer:

    def __init__(self, model: torch.nn.Module, cfg: TrainerConfig, dp_group: Optional[dist.ProcessGroup] = None,
                 pipeline=None):
        """``pipeline``: a :class:`megablocks_b200.parallel.pipeline.PipelineStage` when ``model`` is one
        stage of a pipeline (``TransformerConfig.pipeline_stages > 1``); ``dp_group`` then spans the
        replicas of this stage only."""
        self.model, self.cfg, self.dp_group, self.pipeline = model, cfg, dp_group, pipeline
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
        if cfg.optimizer == 'adafactor':
            opt_cls, kw = Adafactor, dict(lr=cfg.lr, weight_decay=cfg.weight_decay)
        elif cfg.optimizer == 'adam':
            opt_cls, kw = FusedAdam, dict(lr=cfg.lr, betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay)
        else:
            raise ValueError(f"optimizer must be 'adam' or 'adafactor', got {cfg.optimizer!r}")
        if cfg.optimizer != 'adam' and self._update_stream is not None:
            raise ValueError('overlap_expert_update needs the fused Adam optimizer')
        scaling = cfg.loss_scaling if cfg.loss_scaling is not None else params[0].dtype == torch.float16
        self.scaler = DynamicLossScaler(cfg.init_loss_scale, growth_interval=cfg.loss_scale_window) if scaling \
            else None
        if self.world > 1:
            self.flat = FlatBuffer(self.dense_params, granule=self.world * 8)
            self.reducer = GradReducer(self.flat, dp_group, cfg.bucket_mb << 20, shard=cfg.zero1,
                                       backend=cfg.dp_backend)
        # The squared gradient norm is summed over the group by the same peer-memory kernel when the
        # gradients are (one launch, no library collective in the step).
        self._scalar_sum = None
        if self.reducer is not None and self.reducer.backend == 'peer':
            from megablocks_b200.parallel.dp import PeerScalarSum
            self._scalar_sum = PeerScalarSum(dp_group, self.device)
        if self.world > 1 and cfg.zero1:
            # One optimizer "tensor" per owned bucket slice; disjoint across ranks.
            self._shard_params, self._shard_grads = [], []
            for bi in range(len(self.reducer.buckets)):
                lo, hi = self.reducer.shard_range(bi)
                self._shard_params.append(self.flat.param[lo:hi])
                self._shard_grads.append(self.flat.grad[lo:hi])
            self.dense_opt = opt_cls(self._shard_params, **kw)
        else:
            # Replicated tensors: count their norm once across the group.
            self.dense_opt = opt_cls(self.dense_params, norm_weights=[1.0 / self.world] * len(self.dense_params),
                                     **kw)
        self.expert_opt = opt_cls(self.expert_params, **kw)
        self._sqnorm = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.step_count = 0
        self.last_grad_norm = None
        self._h2d = None
        self._norm_sink = None
        if (cfg.fuse_grad_norm and os.environ.get('MB200_FUSE_GRAD_NORM', '1') != '0' and self.device.type == 'cuda' and isinstance(self.expert_opt, FusedAdam)
                and self.expert_params and max(1, int(cfg.grad_accum_steps)) == 1 and pipeline is None):
            from megablocks_b200.ops.gg import GradNormSink
            self._norm_sink = GradNormSink(self.device)
        self._graph = None           # (CUDAGraph, tokens, targets, loss, kernel launches per replay)
        self._eager_steps = 0

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

    def _forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """All micro-batches of one step; returns the mean language-model loss (device scalar)."""
        n = max(1, int(self.cfg.grad_accum_steps))
        scale = (self.scaler.scale if self.scaler is not None else 1.0) / n
        if self.pipeline is not None:
            return self._pipeline_forward_backward(tokens, targets, n, scale)
        if n == 1:
            with nvtx_range('forward'):
                total, lm = self.model.loss(tokens, targets)
            with nvtx_range('backward'):
                (total if scale == 1.0 else total * scale).backward()
            return lm
        if tokens.shape[0] % n:
            raise ValueError(f'batch of {tokens.shape[0]} rows does not split into {n} micro-batches')
        lm_sum = None
        for i, (tok, tgt) in enumerate(zip(tokens.chunk(n), targets.chunk(n))):
            if self.reducer is not None:
                self.reducer.active = i == n - 1
            with nvtx_range('forward'):
                total, lm = self.model.loss(tok, tgt)
            with nvtx_range('backward'):
                (total * scale).backward()
            lm_sum = lm if lm_sum is None else lm_sum + lm
        if self.reducer is not None:
            self.reducer.active = True
        return lm_sum / n

    def _pipeline_forward_backward(self, tokens, targets, n: int, scale: float) -> torch.Tensor:
        """One step of a pipeline stage: ``n`` micro-batches through ``PipelineStage.forward_backward``.

        Every stage gets the same ``tokens`` / ``targets`` (the first uses the tokens, the last the
        targets).  Each micro-batch adds this stage's own load-balancing terms to what it
        back-propagates, which is why a stage must have collected exactly ``num_layers /
        pipeline stages`` of them (the rule megablocks/layers/moe.py:39-60 checks).
        """
        stage = self.pipeline
        if tokens.shape[0] % n:
            raise ValueError(f'batch of {tokens.shape[0]} rows does not split into {n} micro-batches')
        tok_chunks, tgt_chunks = tokens.chunk(n), targets.chunk(n)
        lm_values = []

        def run_stage(x, index):
            return self.model.stage_forward(tok_chunks[index] if stage.is_first else x)

        def loss_fn(hidden, index):
            lm = self.model.stage_loss(hidden, tgt_chunks[index])
            lm_values.append(lm.detach())
            return lm

        if self.reducer is not None:
            self.reducer.active = False      # the schedule interleaves micro-batches: reduce once, at the end
        stage.forward_backward(run_stage, n, loss_fn, scale=scale)
        if self.reducer is not None:
            self.reducer.active = True
        if lm_values:
            return torch.stack(lm_values).mean()
        return torch.zeros((), device=self.device)

    # -- whole-step CUDA graph ---------------------------------------------------------
    def _graph_eligible(self) -> bool:
        # Several ranks: the kernels of the fused expert-parallel exchange and of the peer-memory
        # gradient reducer take their sequence numbers from device counters that the recorded step
        # advances itself; NCCL-backed reducers and ZeRO-1 keep host-side state per step.
        multi_ok = self.world == 1 or (self.reducer is not None and self.reducer.backend == 'peer'
                                       and not self.cfg.zero1)
        return (self.cfg.cuda_graph and self.device.type == 'cuda' and multi_ok and self.pipeline is None
                and self.scaler is None and self._update_stream is None
                and isinstance(self.dense_opt, FusedAdam) and isinstance(self.expert_opt, FusedAdam)
                and self.step_count <= max(int(self.cfg.total_steps), 1))     # rows of the schedule table

    def _hyper_table(self) -> torch.Tensor:
        """Row ``s`` = {learning rate, bias1, bias2} of the step taken when ``step_count == s``."""
        cfg = self.cfg
        rows = max(int(cfg.total_steps), 1) + 1
        b1, b2 = cfg.betas
        steps = torch.arange(rows, dtype=torch.float64)
        lr = torch.tensor([cosine_lr(s, cfg.total_steps, cfg.lr, cfg.min_lr, cfg.warmup_fraction) if cfg.schedule
                           else cfg.lr for s in range(rows)], dtype=torch.float64)
        table = torch.stack([lr, 1.0 - b1**(steps + 1), 1.0 - b2**(steps + 1)], dim=1)
        return table.float().to(self.device)

    def _capture(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        from megablocks_b200._ext import ext
        assert self.dense_opt.step_count == self.step_count and self.expert_opt.step_count == self.step_count
        self._table = self._hyper_table()
        self._graph_step = torch.tensor([self.step_count], dtype=torch.int64, device=self.device)
        self._hyper = torch.zeros(3, dtype=torch.float32, device=self.device)
        self.dense_opt.hyper = self.expert_opt.hyper = self._hyper
        static_tokens, static_targets = tokens.clone(), targets.clone()
        self._zero_grad()
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()     # the graph gets a pool of its own: hand back what the warm-up steps cached
        graph = torch.cuda.CUDAGraph()
        before = ext().launch_count()
        counters = (self.step_count, self.dense_opt.step_count, self.expert_opt.step_count)
        # Sequence numbers of the peer-memory exchanges: the recorded launches keep the numbers the
        # host hands out now, and the step ends by adding "uses per step" to each user's device
        # counter, which every kernel adds to its number: replay r runs with the numbers the r-th
        # step after this one would have had.
        from megablocks_b200.parallel.ep import live_workspaces
        users = [u for u in live_workspaces() + [self.reducer, self._scalar_sum]
                 if u is not None and hasattr(u, 'seq_dev')]
        marks = [(u, u.seq, getattr(u, 'released_seq', None)) for u in users]
        try:
            # Other threads (a process group's watchdog polling its events) must stay free to make
            # CUDA calls that are not part of the recording.
            mode = dict(capture_error_mode='thread_local') if self.world > 1 else {}
            with torch.cuda.graph(graph, **mode):
                torch.index_select(self._table, 0, self._graph_step, out=self._hyper.view(1, 3))
                self._graph_step.add_(1)
                if self.flat is not None:
                    self.flat.zero_grad()
                loss = self._step_eager(static_tokens, static_targets, zero_grad=False)
                for user, seq, _ in marks:
                    if user.seq != seq:
                        user.seq_dev.add_(user.seq - seq)
        finally:
            # Recording advanced the host-side counters without running anything: take that back.
            # (Also the sequence numbers: replay r runs with "recorded number + r - 1", so a step
            # launched kernel by kernel after R replays must get "recorded number + R", which is
            # what the host's next number plus the device counter gives once the host is back at
            # its value from before the recording.)
            self.step_count, self.dense_opt.step_count, self.expert_opt.step_count = counters
            for user, seq, released in marks:
                user.seq = seq
                if released is not None:
                    user.released_seq = released
        launches = ext().launch_count() - before
        self._graph = (graph, static_tokens, static_targets, loss, launches)

    def _graph_replay(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        from megablocks_b200._ext import ext
        graph, static_tokens, static_targets, loss, launches = self._graph
        static_tokens.copy_(tokens, non_blocking=True)
        static_targets.copy_(targets, non_blocking=True)
        graph.replay()
        ext().count_launches(launches)
        cfg = self.cfg        # the kernels read the rate from the device table; keep the host's copy for logs
        self.dense_opt.lr = self.expert_opt.lr = cosine_lr(
            self.step_count, cfg.total_steps, cfg.lr, cfg.min_lr, cfg.warmup_fraction) if cfg.schedule else cfg.lr
        self.step_count += 1
        self.dense_opt.step_count += 1
        self.expert_opt.step_count += 1
        return loss.clone()

    def drop_graph(self) -> None:
        """Forget the recorded step (before changing the model, the optimizers or the batch shape)."""
        self._graph = None
        self._eager_steps = 0
        if isinstance(self.dense_opt, FusedAdam):
            self.dense_opt.hyper = None
        if isinstance(self.expert_opt, FusedAdam):
            self.expert_opt.hyper = None

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Forward, backward, gradient reduction, clipping and the optimizer update.

        ``tokens`` / ``targets`` hold this rank's whole share of the step: ``grad_accum_steps``
        micro-batches stacked along dimension 0.  Returns the language-model loss as a device
        scalar (no host sync, except under fp16 loss scaling, which reads one overflow flag).

        With ``cfg.cuda_graph`` the first ``graph_warmup_steps`` calls run kernel by kernel, the next
        one records the step in a CUDA graph, and every call from then on copies the batch into the
        graph's input buffers and replays it.
        """
        if self._graph_eligible():
            if self._graph is not None:
                _, static_tokens, _, _, _ = self._graph
                if static_tokens.shape != tokens.shape:
                    self.drop_graph()
            if self._graph is None and self._eager_steps >= self.cfg.graph_warmup_steps:
                failed = None
                try:
                    self._capture(tokens, targets)
                except RuntimeError as err:      # something in the step cannot be recorded: stay kernel by kernel
                    failed = err
                if self.world > 1:
                    # Recording takes a different time on every rank (and may fail on one only): the
                    # ranks meet here, so that the bounded device waits of the step that follows do
                    # not have to absorb the difference.
                    torch.cuda.synchronize(self.device)
                    dist.barrier(self.dp_group)
                if failed is not None:
                    import warnings
                    warnings.warn(f'CUDA-graph capture of the training step failed, continuing without: {failed}')
                    self.drop_graph()
                    self.cfg = dataclasses.replace(self.cfg, cuda_graph=False)
                    # The abandoned recording may have stopped anywhere: bring the per-step host state
                    # back to "no step in progress".
                    if self.reducer is not None:
                        self.reducer.reset()
                    from megablocks_b200.layers.moe import clear_load_balancing_loss
                    from megablocks_b200.layers.router import clear_router_zloss
                    clear_load_balancing_loss()
                    clear_router_zloss()
                    self._zero_grad()
                    return self._step_eager(tokens, targets)
            if self._graph is not None:
                return self._graph_replay(tokens, targets)
            self._eager_steps += 1
        elif self._graph is not None:
            self.drop_graph()        # past the end of the schedule table: back to plain launches
        return self._step_eager(tokens, targets)

    def _step_eager(self, tokens: torch.Tensor, targets: torch.Tensor, zero_grad: bool = True) -> torch.Tensor:
        cfg = self.cfg
        self.model.train()
        if zero_grad:
            self._zero_grad()
        sink = self._norm_sink
        if sink is not None:
            from megablocks_b200.ops import gg
            sink.begin()
            gg.set_grad_norm_sink(sink)
            try:
                lm = self._forward_backward(tokens, targets)
            finally:
                gg.set_grad_norm_sink(None)
        else:
            lm = self._forward_backward(tokens, targets)
        with nvtx_range('grad_reduce_wait'):
            if self.reducer is not None:
                self.reducer.finish()
        lr = cosine_lr(self.step_count, cfg.total_steps, cfg.lr, cfg.min_lr, cfg.warmup_fraction) if cfg.schedule \
            else cfg.lr
        self.dense_opt.lr = self.expert_opt.lr = lr

        dense_grads = self._shard_grads if (self.world > 1 and cfg.zero1) else None
        self.flush()   # a layer that did not run this step may still have an update in flight
        with nvtx_range('grad_norm'):
            self._sqnorm.zero_()
            self.dense_opt.add_sqnorm(self._sqnorm, dense_grads)
            if sink is not None:
                # Gradients that are exactly the output of a weight-gradient GEMM already have their
                # sum of squares in a slot of the sink; the rest is summed by the kernel.
                slots = [sink.lookup(g) if w == 1.0 else None
                         for g, w in zip(self.expert_opt.grads(), self.expert_opt.norm_weights)]
                self.expert_opt.add_sqnorm(self._sqnorm, skip=[s is not None for s in slots])
                found = [s for s in slots if s is not None]
                self.fused_norm_tensors = len(found)
                if found:
                    lo, hi = min(found), max(found) + 1
                    if hi - lo == len(set(found)) == len(found):       # a run of slots, in any order
                        self._sqnorm += sink.slots[lo:hi].sum()
                    else:
                        key = tuple(found)
                        if getattr(self, '_slot_key', None) != key:    # the same launches every step: built once
                            self._slot_key = key
                            self._slot_index = torch.tensor(found, dtype=torch.int64, device=self.device)
                        self._sqnorm += sink.slots.index_select(0, self._slot_index).sum()
            else:
                self.expert_opt.add_sqnorm(self._sqnorm)
            if self.world > 1:
                if self._scalar_sum is not None:
                    self._scalar_sum(self._sqnorm)
                else:
                    dist.all_reduce(self._sqnorm, group=self.dp_group)
            if self.pipeline is not None and self.pipeline.world > 1:
                dist.all_reduce(self._sqnorm, group=self.pipeline.group)
        extra = 1.0
        if self.scaler is not None:
            # The squared norm was summed over every rank, so all ranks take the same decision.
            overflow = not bool(torch.isfinite(self._sqnorm).all().item())
            scale = self.scaler.scale
            self.scaler.update(overflow)
            if overflow:          # skip the update; the next step retries with a smaller scale
                self.last_grad_norm = self._sqnorm.sqrt()
                return lm
            self._sqnorm.div_(scale * scale)
            extra = 1.0 / scale
        coeff = clip_coefficient(self._sqnorm, cfg.max_grad_norm, extra)
        self.last_grad_norm = coeff[1:2]
        with nvtx_range('optimizer'):
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

    def run_from_host(self, batches) -> list:
        """Train one step per pinned host batch (``[micro_batch, seq + 1]`` int64 each) and return
        every step's loss as a Python float, in order.

        Each step copies its own batch to the device and its loss is copied back to pinned host
        memory; the host waits for the loss of step ``k`` only after it has queued step ``k + 1``,
        so the device never idles while the host reads a number and prepares the next launch.
        """
        losses, pending = [], None
        pinned = self.device.type == 'cuda'
        if self._h2d is None:       # allocated once: pinning memory is slow and synchronises the device
            self._h2d = ([torch.empty(1, dtype=torch.float32, pin_memory=pinned) for _ in range(2)],
                         [torch.cuda.Event() for _ in range(2)] if pinned else [None, None])
        ring, events = self._h2d

        def collect(slot):
            if events[slot] is not None:
                events[slot].synchronize()
            losses.append(float(ring[slot][0]))

        for i, batch in enumerate(batches):
            dev = batch.to(self.device, non_blocking=True)
            loss = self.step(dev[:, :-1], dev[:, 1:])
            slot = i & 1
            ring[slot].copy_(loss.detach().float().reshape(1), non_blocking=True)
            if events[slot] is not None:
                events[slot].record()
            if pending is not None:
                collect(pending)
            pending = slot
        if pending is not None:
            collect(pending)
        return losses

    def state_dict(self):
        self.flush()
        state = {'model': self.model.state_dict(), 'dense_opt': self.dense_opt.state_dict(),
                 'expert_opt': self.expert_opt.state_dict(), 'step': self.step_count}
        state['opt_layout'] = self._opt_layout()
        if self.scaler is not None:
            state['loss_scaler'] = self.scaler.state_dict()
        return state

    def _opt_groups(self):
        """(optimizer, its tensors) for the optimizers whose flat state is laid out per parameter."""
        groups = []
        if isinstance(self.expert_opt, FusedAdam):
            groups.append(('expert_opt', self.expert_opt, self.expert_params))
        if isinstance(self.dense_opt, FusedAdam) and not (self.world > 1 and self.cfg.zero1):
            groups.append(('dense_opt', self.dense_opt, self.dense_params))
        return groups

    def _opt_layout(self):
        """Where every named parameter's Adam state sits in the flat buffers: ``{optimizer: [(name,
        offset, shape)]}``.  With it a checkpoint can be converted to another expert-parallel degree
        (:func:`megablocks_b200.checkpoint.load`): the state is cut out per parameter and resharded
        by the same rule as the weights.  ZeRO-sharded and Adafactor state has no such layout and is
        left out (it restarts after a change of degree)."""
        names = {id(p): n for n, p in self.model.named_parameters()}
        return {key: [(names[id(p)], off, list(p.shape)) for p, off in zip(opt.params, opt.offsets)]
                for key, opt, _ in self._opt_groups()}

    def _load_named_opt_state(self, named, step):
        names = {id(p): n for n, p in self.model.named_parameters()}
        for _, opt, _ in self._opt_groups():
            for p, off in zip(opt.params, opt.offsets):
                n, entry = p.numel(), named.get(names[id(p)])
                if entry is None:      # no state for this tensor: keep the loaded weights, restart the moments
                    opt.master[off:off + n].copy_(p.detach().reshape(-1))
                    opt.exp_avg[off:off + n].zero_()
                    opt.exp_avg_sq[off:off + n].zero_()
                    continue
                for part in ('master', 'exp_avg', 'exp_avg_sq'):
                    getattr(opt, part)[off:off + n].copy_(entry[part].reshape(-1))
                p.data.copy_(opt.master[off:off + n].view_as(p))
            opt.step_count = int(step)

    def load_state_dict(self, state):
        self.flush()
        self.drop_graph()            # the recorded step counts from the old step number
        self.model.load_state_dict(state['model'])
        if 'dense_opt' in state and 'expert_opt' in state:
            self.dense_opt.load_state_dict(state['dense_opt'])
            self.expert_opt.load_state_dict(state['expert_opt'])
        else:
            # Weights only, or written at another expert-parallel degree and converted by
            # checkpoint.load: the master copies follow the loaded weights, then whatever
            # per-parameter state the checkpoint carries is put in place.
            self.dense_opt.resync_master()
            self.expert_opt.resync_master()
            if 'opt_named' in state:
                self._load_named_opt_state(state['opt_named'], state.get('opt_step', state.get('step', 0)))
        self.step_count = int(state.get('step', 0))
        if self.scaler is not None and 'loss_scaler' in state:
            self.scaler.load_state_dict(state['loss_scaler'])


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
    from megablocks_b200.layers.moe import ParallelMLP
    from megablocks_b200.parallel.pipeline import PipelineStage
    from megablocks_b200.utils.metrics import JsonlLogger, expert_load_stats

    ap = argparse.ArgumentParser(description='Train a dMoE / MoE transformer on synthetic tokens.')
    ap.add_argument('--preset', choices=sorted(PRESETS), default='dmoe-125m')
    ap.add_argument('--micro-batch', type=int, default=32)
    ap.add_argument('--global-batch', type=int, default=None,
                    help='sequences per optimizer step over all data-parallel ranks; the step then runs '
                         'global / (micro x data-parallel ranks) micro-batches with gradient accumulation')
    ap.add_argument('--precision', choices=['bf16', 'fp16'], default='bf16',
                    help='fp16 trains under dynamic loss scaling')
    ap.add_argument('--optimizer', choices=['adam', 'adafactor'], default='adam')
    ap.add_argument('--pp', type=int, default=1, help='pipeline stages (ranks are split stage-major)')
    ap.add_argument('--init-std', type=float, default=None)
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
    ap.add_argument('--dp-comm', choices=['auto', 'peer', 'nccl'], default='auto',
                    help='gradient reduction of the replicated parameters: own peer-memory kernel or NCCL')
    ap.add_argument('--cuda-graph', dest='cuda_graph', action='store_true',
                    help='record the whole step in one CUDA graph after three ordinary steps and replay it '
                         '(bf16 / fp32, fused Adam, no pipeline stages, no ZeRO-1, peer-memory gradient reducer)')
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
    pp = max(1, args.pp)
    if world % pp:
        raise SystemExit(f'--pp {pp} does not divide the {world} ranks')
    dp_world = world // pp            # ranks per stage: data parallel for dense, expert parallel for MoE weights
    stage_index, stage_rank = rank // dp_world, rank % dp_world
    pp_group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29500')
        dist.init_process_group('nccl' if use_cuda else 'gloo', rank=rank, world_size=world)
        group = dist.group.WORLD
        if pp > 1:
            # Every rank creates every group, in the same order.
            stage_groups = [dist.new_group(list(range(s * dp_world, (s + 1) * dp_world))) for s in range(pp)]
            chain_groups = [dist.new_group([s * dp_world + r for s in range(pp)]) for r in range(dp_world)]
            group = stage_groups[stage_index] if dp_world > 1 else None
            pp_group = chain_groups[stage_rank]

    torch.manual_seed(args.seed)
    overrides = dict(device=device, expert_parallel_group=group, mlp_impl=args.mlp_impl,
                     moe_loss_weight=args.loss_weight, activation_checkpointing=args.recompute,
                     ep_fused_comm={'auto': None, 'fused': True, 'nccl': False}[args.ep_comm],
                     dtype=(torch.float16 if args.precision == 'fp16' else torch.bfloat16) if use_cuda
                     else torch.float32,
                     pipeline_stages=pp, pipeline_stage=stage_index)
    if args.init_std is not None:
        overrides['init_std'] = args.init_std
    accum = 1
    if args.global_batch is not None:
        per_pass = args.micro_batch * dp_world
        if args.global_batch % per_pass:
            raise SystemExit(f'--global-batch {args.global_batch} is not a multiple of micro-batch x '
                             f'data-parallel ranks = {per_pass}')
        accum = args.global_batch // per_pass
    if pp > 1:
        overrides['ep_inflight_microbatches'] = accum      # all forwards of a step precede its backwards
    if args.experts is not None:
        overrides['moe_num_experts'] = args.experts
    if args.top_k is not None:
        overrides['moe_top_k'] = args.top_k
    if args.capacity_factor is not None:
        overrides.update(dropless=False, moe_capacity_factor=args.capacity_factor)
    cfg = preset(args.preset, **overrides)
    model = MoETransformer(cfg)
    stage = None
    if pp > 1:
        stage = PipelineStage(pp_group, (args.micro_batch, cfg.max_seq_len, cfg.hidden_size), cfg.dtype, device)
    trainer = Trainer(model, TrainerConfig(lr=args.lr, min_lr=args.min_lr, total_steps=args.steps, zero1=args.zero1,
                                           overlap_expert_update=args.defer_expert_update, dp_backend=args.dp_comm,
                                           grad_accum_steps=accum, optimizer=args.optimizer,
                                           cuda_graph=args.cuda_graph),
                      dp_group=group, pipeline=stage)
    if args.load:
        state = checkpoint.load(args.load, rank, world, map_location=device)
        trainer.load_state_dict(state)
    # The loss lives on the last pipeline stage: its first rank reports.
    reporter = stage_index == pp - 1 and stage_rank == 0
    logger = JsonlLogger(args.log, 0 if reporter else 1)
    heartbeat = Heartbeat(timeout_s=60.0) if world > 1 else None
    # Ranks of one pipeline chain must draw the same batch (first stage: tokens, last stage: targets).
    gen = torch.Generator().manual_seed(args.seed + stage_rank)
    rows = args.micro_batch * accum
    tokens_per_step = dp_world * rows * cfg.max_seq_len
    moe_layers = [m for m in model.modules() if isinstance(m, ParallelMLP)]
    t_last, loss = time.time(), None
    for step in range(trainer.step_count, args.steps):
        if heartbeat is not None:
            heartbeat.check()
        batch = synthetic_batch(rows, cfg.max_seq_len, cfg.vocab_size, gen)
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
            load = {}
            for i, layer in enumerate(moe_layers):       # per-layer expert load of the last micro-batch
                tpe = getattr(layer, 'last_tokens_per_expert', None)
                if tpe is not None:
                    load[f'layer{i}'] = expert_load_stats(tpe)
            logger.log(step=step + 1, loss=value, grad_norm=trainer.last_grad_norm, tokens_per_s=rate,
                       lr=trainer.dense_opt.lr, expert_load=load,
                       loss_scale=trainer.scaler.scale if trainer.scaler is not None else None,
                       skipped_steps=trainer.scaler.skipped_steps if trainer.scaler is not None else 0)
            if reporter:
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
