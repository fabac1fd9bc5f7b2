"""Training / evaluation loops (``recis/framework/trainer.py:26-397``).

Same constructor, ``TrainingArguments`` and loop structure as the reference (zero_grad -> forward -> backward -> dense step
-> sparse step -> scheduler; hooks after every step; periodic + final checkpoint; cooperative end-of-data). Differences:
* data parallelism of the dense tower uses ``DenseGradReducer`` (one flat gradient buffer, averaged by our peer-memory
  all-reduce kernel on CUDA, overlapped with the sparse update) instead of HF accelerate + DistributedDataParallel;
* the end-of-data flag is exchanged every ``stop_check_interval`` steps (default 1 = the reference's behaviour) and only
  when more than one rank runs, so a single-GPU loop never synchronises with the host;
* ``train_steps`` steps are executed (the reference stops one short, ``trainer.py:359``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from ..hooks import Hook, LoggerHook
from ..parallel.dense_reducer import DenseGradReducer
from ..utils.data_utils import copy_data_to_device
from ..utils.logger import Logger
from .checkpoint_manager import CheckpointManager, Saver
from .metrics import get_global_metrics

logger = Logger(__name__)


@dataclass
class TrainingArguments:
    gradient_accumulation_steps: int = 1
    output_dir: str = "output_dir"
    model_bank: Optional[list] = None
    log_steps: int = 100
    train_steps: Optional[int] = None
    train_epoch: Optional[int] = 1
    eval_steps: Optional[int] = None
    save_steps: Optional[int] = 1000
    max_to_keep: int = 5
    save_concurrency_per_rank: int = 4
    stop_check_interval: int = 1
    max_empty_windows: int = 1000      # windowed datasets: this many empty windows in a row end the data (streams have no last window)
    heartbeat_timeout: float = 0.0     # > 0: ranks exchange heartbeats; a peer silent for this many seconds raises PeerLostError


class Trainer:
    def __init__(self, model: Optional[nn.Module] = None, args: TrainingArguments = None, train_dataset=None, eval_dataset=None,
                 hooks: Optional[List[Hook]] = None, dense_optimizers: Tuple = (None, None), sparse_optimizer=None,
                 data_to_cuda: bool = False, **kwargs) -> None:
        self.args = args or TrainingArguments()
        self.hooks = list(hooks or [])
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.model = model
        self.dense_optimizer, self.dense_lr_scheduler = dense_optimizers
        self.sparse_optimizer = sparse_optimizer
        self.data_to_cuda = data_to_cuda
        self.gradient_accumulation_steps = max(int(self.args.gradient_accumulation_steps), 1)
        self.world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        self.reducer = None
        if self.world > 1 and self.dense_optimizer is not None:
            params = [p for g in self.dense_optimizer.param_groups for p in g["params"] if p.requires_grad]
            if params:
                # every rank starts from rank 0's dense weights, as DistributedDataParallel does at construction (the reference
                # wraps the model in DDP, recis/framework/trainer.py:170-184); buffers are included
                with torch.no_grad():
                    for t in list(model.parameters()) + list(model.buffers()):
                        if t.is_floating_point() or t.dtype in (torch.int32, torch.int64, torch.bool, torch.uint8):
                            dist.broadcast(t.data, src=0)
                self.reducer = DenseGradReducer(params, self.world)
        if self.sparse_optimizer is not None:
            self.sparse_optimizer.set_grad_accum_steps(self.gradient_accumulation_steps)
        self._global_step = torch.scalar_tensor(0, dtype=torch.int64)
        self._micro_step = 0
        self.build_checkpoint_manager(model, self.args)
        self.has_restore = False
        self.hooks.append(LoggerHook(self.args.log_steps))
        self._device = next((p.device for p in model.parameters()), torch.device("cpu")) if model is not None else torch.device("cpu")
        self.stop_state = torch.zeros((), dtype=torch.int64, device=self._device if self._device.type == "cuda" else "cpu")
        self.peer_monitor = None
        if self.world > 1 and self.args.heartbeat_timeout > 0:
            from .health import PeerMonitor
            self.peer_monitor = PeerMonitor(dist.get_rank(), self.world, interval=min(1.0, self.args.heartbeat_timeout / 4),
                                            timeout=self.args.heartbeat_timeout).start()

    # ---- checkpointing
    def build_saver(self, model, args):
        return Saver(model, self.sparse_optimizer, output_dir=args.output_dir, max_keep=args.max_to_keep,
                     concurrency=args.save_concurrency_per_rank)

    def build_checkpoint_manager(self, model, args):
        saver = self.build_saver(model, args)
        self.checkpoint_manager = CheckpointManager(saver=saver, save_interval=args.save_steps)
        if self.train_dataset is not None and hasattr(self.train_dataset, "dump_io_state"):
            saver.register_io_state("train_io", self.train_dataset)
        # a windowed dataset's position (which window comes next) is saved with the checkpoint and restored with it
        # (``recis/framework/trainer.py:199-208``)
        if self._windowed(self.train_dataset):
            saver.register_for_checkpointing("train_window_io", self.train_dataset)
        if self._windowed(self.eval_dataset):
            saver.register_for_checkpointing("eval_window_io", self.eval_dataset)
        if self.dense_optimizer is not None:
            saver.register_for_checkpointing("dense_optimizer", self.dense_optimizer)
        if self.dense_lr_scheduler is not None:
            saver.register_for_checkpointing("dense_lr_scheduler", self.dense_lr_scheduler)

    def add_hooks(self, hooks: List[Hook]):
        for hook in hooks:
            self.add_hook(hook)

    def add_hook(self, hook: Hook):
        self.hooks.append(hook)

    def restore(self):
        if not self.has_restore:
            self.checkpoint_manager.load_model_bank(self.args.model_bank)
            self._global_step = self.checkpoint_manager.restore()
            self.has_restore = True

    # ---- loops
    def train(self, train_steps=None):
        self.restore()
        for hook in self.hooks:
            hook.before_train()
        for epoch in range(self.args.train_epoch or 1):
            if epoch > 0 and self._windowed(self.train_dataset) and hasattr(self.train_dataset, "reset"):
                self.train_dataset.reset()          # a further epoch starts at the first window again
            for hook in self.hooks:
                hook.before_epoch()
            self._train_loop(self.args.train_steps if train_steps is None else train_steps, epoch=epoch)
            for hook in self.hooks:
                hook.after_epoch()
        for hook in self.hooks:
            hook.after_train()
            hook.end()

    def train_and_evaluate(self, epochs=1, train_steps=None, eval_steps=None):
        self.restore()
        for epoch in range(epochs):
            self._train_loop(self.args.train_steps if train_steps is None else train_steps, epoch=epoch)
            self.evaluate(eval_steps=eval_steps, _end_hooks=False)
        for hook in self.hooks:
            hook.end()

    def sync_exit_flag(self, flag: bool) -> bool:
        if self.world == 1:
            return flag
        self.stop_state.fill_(int(flag))
        dist.all_reduce(self.stop_state, op=dist.ReduceOp.MAX)
        return bool(self.stop_state.item())

    @staticmethod
    def _next(iterator):
        """Datasets yield ``(stop_flag, batch)``; a plain iterable of batches is accepted too."""
        try:
            item = next(iterator)
        except StopIteration:
            return True, None
        if isinstance(item, tuple) and len(item) == 2 and isinstance(item[0], (bool, int)):
            return bool(item[0]), item[1]
        return False, item

    # ---- windowed datasets (``next_window()`` until StopIteration; ``recis/framework/trainer.py:322-345``)
    @staticmethod
    def _windowed(dataset) -> bool:
        return dataset is not None and hasattr(dataset, "next_window")

    def get_new_window_iter(self, dataset):
        """Iterator over the next window that has data, or None when the dataset has no further window. A stream has no last
        window: after ``max_empty_windows`` (a ``TrainingArguments`` field or 1000) empty ones in a row the data is taken to
        have ended rather than skipping ahead for ever."""
        if not self._windowed(dataset):
            raise TypeError("dataset must be window_io")
        limit = int(getattr(self.args, "max_empty_windows", 1000) or 1000)
        empty = 0
        while True:
            try:
                need_skip = dataset.next_window()
            except StopIteration:
                logger.info("Window IO Finish")
                return None
            offset = int(dataset._read_offset[0]) if hasattr(dataset, "_read_offset") else -1
            if not need_skip:
                logger.info(f"Next window, offset = {offset}")
                return iter(dataset)
            logger.info(f"Skip for window, offset = {offset}")
            empty += 1
            if empty >= limit:
                logger.warning(f"{empty} empty windows in a row: treating the data as finished")
                return None

    def _first_iter(self, dataset):
        return self.get_new_window_iter(dataset) if self._windowed(dataset) else iter(dataset)

    def _next_of(self, dataset, iterator):
        """``(stop, batch, iterator)``: the next batch, moving on to the dataset's next window when the current one ends."""
        while True:
            stop, data = (True, None) if iterator is None else self._next(iterator)
            if not stop or not self._windowed(dataset) or iterator is None:
                return stop, data, iterator
            iterator = self.get_new_window_iter(dataset)

    def evaluate(self, eval_steps=None, _end_hooks=True):
        self.restore()
        iterator = self._first_iter(self.eval_dataset)
        eval_steps = self.args.eval_steps if eval_steps is None else eval_steps
        lstep = 0
        for hook in self.hooks:
            hook.before_evaluate()
        self.model.eval()
        while eval_steps is None or lstep < eval_steps:
            stop, data, iterator = self._next_of(self.eval_dataset, iterator)
            if self.sync_exit_flag(stop):
                break
            if self.data_to_cuda:
                data = copy_data_to_device(data, "cuda")
            with torch.no_grad():
                self.model(data)
            metrics = dict(get_global_metrics())
            for hook in self.hooks:
                hook.after_step(metrics, self._global_step)
            lstep += 1
        for hook in self.hooks:
            hook.after_evaluate()
            if _end_hooks:
                hook.end()

    def _train_loop(self, max_steps=None, epoch=1):
        self.model.train()
        iterator = self._first_iter(self.train_dataset)
        lstep = 0
        check = max(int(self.args.stop_check_interval), 1)
        while max_steps is None or lstep < max_steps:
            stop, data, iterator = self._next_of(self.train_dataset, iterator)
            if lstep % check == 0 or stop:
                stop = self.sync_exit_flag(stop)
            if stop:
                break
            if self.data_to_cuda:
                data = copy_data_to_device(data, "cuda")
            if self.peer_monitor is not None:
                self.peer_monitor.check()          # a dead or stalled peer surfaces here, before kernels that would wait for it
            for hook in self.hooks:
                hook.before_step()
            metrics = {}
            self._train_step(data, epoch, metrics)
            for hook in self.hooks:
                hook.after_step(metrics, self._global_step)
            self.checkpoint_manager.step()
            self._global_step = self.checkpoint_manager.global_step
            lstep += 1
            if lstep % max(int(self.args.log_steps), 1) == 0:
                self.check_communication()
        self.check_communication()
        self.checkpoint_manager.save()

    def check_communication(self):
        """Read the status words of the fused exchanges and of the dense all-reduce (one small host read each) and raise if a
        bounded wait ran out or an exchange window overflowed. Called every ``log_steps`` steps and before the final save, so that
        such a condition ends the run with an error instead of training on with dropped rows."""
        seen = set()
        for m in self.model.modules():
            ex = getattr(m, "fused", None)
            if ex is not None and id(ex) not in seen and hasattr(ex, "check"):
                seen.add(id(ex))
                ex.check()
        if self.reducer is not None:
            self.reducer.check()

    def _train_step(self, data, epoch, metrics):
        accum = self.gradient_accumulation_steps
        boundary = (self._micro_step + 1) % accum == 0
        if self._micro_step % accum == 0:
            if self.dense_optimizer is not None:
                self.dense_optimizer.zero_grad(set_to_none=self.reducer is None)
        if self.sparse_optimizer is not None:
            self.sparse_optimizer.zero_grad()
        loss = self.model(data)
        if isinstance(loss, (tuple, list)):
            loss = loss[0]
        metrics.update(epoch=epoch, loss=loss.detach())
        metrics.update(get_global_metrics())
        # Every micro-batch back-propagates its unscaled loss. At the boundary both parameter kinds see the MEAN over the
        # micro-batches: the sparse optimizer divides its staged gradients by the accumulation count itself
        # (set_grad_accum_steps), the dense gradients are divided here. (The reference sums the dense gradients and averages
        # the sparse ones, recis/framework/trainer.py:383-397 with csrc/embedding/hashtable.cc:129.)
        if self.reducer is not None:
            # buckets of dense gradients start their average from backward's hooks, at accumulation boundaries only; the
            # division by the accumulation count is folded into the average
            self.reducer.armed = boundary
            self.reducer.grad_scale = 1.0 / accum
        loss.backward()
        if boundary and accum > 1 and self.dense_optimizer is not None and self.reducer is None:
            grads = [p.grad for g in self.dense_optimizer.param_groups for p in g["params"] if p.grad is not None]
            if grads:
                torch._foreach_mul_(grads, 1.0 / accum)
        if boundary and self.reducer is not None:
            self.reducer.all_reduce_async()
        if self.sparse_optimizer is not None:
            self.sparse_optimizer.step()
        if boundary:
            if self.reducer is not None:
                self.reducer.wait()
            if self.dense_optimizer is not None:
                self.dense_optimizer.step()
            if self.dense_lr_scheduler is not None:
                self.dense_lr_scheduler.step()
        self._micro_step += 1
