"""Checkpoint saving / restoring around the training loop (``recis/framework/checkpoint_manager.py:24-505``).

Directory layout (same as the reference):
``<output_dir>/checkpoint`` (one checkpoint id per line), ``<output_dir>/ckpt_<step>/`` holding the sparse bundle
(``model-*.safetensors``, ``index``, ``tensorkey.json``, ``torch_rank_weights_embs_table_multi_shard.json``),
``model.pt`` (dense state dict), ``extra.pt`` (registered extras incl. ``global_step`` and the dense optimizer),
``io_state_<rank>.pt`` + ``io_state_count``. ``load_by_config`` takes ``{"load": [...], "exclude": [...], "strict": bool}``
over the parts ``sparse, dense, extra, sparse_opt, io_state``.

``output_dir`` (and a model-bank ``path``) may also be a URL of any file system that fsspec knows (``hdfs://``, ``s3://``,
``memory://`` ...); the reference routes its Python-side files through fsspec but registers the local file system only
(``recis/framework/filesystem.py:18-64``). The native writers and readers work on local files, so a remote directory is served
through a staging directory (``$RECIS_STAGING_DIR`` or a temporary one, one sub-directory per rank): a checkpoint is written
there, every rank uploads the files it wrote, rank 0 uploads the ``checkpoint`` listing last (after a barrier), and pruned
checkpoints are removed remotely as well; loading downloads the listing and the wanted checkpoint first.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import tempfile
from typing import Optional

import torch
import torch.distributed as dist

from ..nn.modules.hashtable import split_sparse_dense_state_dict
from ..serialize import Loader as SLoader, Saver as SSaver
from ..utils.logger import Logger
from ..utils.mos import Mos

logger = Logger(__name__)


def _is_remote(path) -> bool:
    p = str(path)
    return "://" in p and not p.startswith("file://")


def _remote_fs(url: str):
    import fsspec
    fs, root = fsspec.core.url_to_fs(str(url))
    return fs, root.rstrip("/")


_STAGING = None


def _staging_root() -> str:
    """Local directory that stands in for remote ones, one per rank and process tree: ``$RECIS_STAGING_DIR/rank<r>`` or a
    temporary directory."""
    global _STAGING
    if _STAGING is None:
        base = os.environ.get("RECIS_STAGING_DIR")
        rank = os.environ.get("RANK", "0")
        if base:
            _STAGING = os.path.join(base, f"rank{rank}")
            os.makedirs(_STAGING, exist_ok=True)
        else:
            _STAGING = tempfile.mkdtemp(prefix=f"recis_staging_rank{rank}_")
    return _STAGING


class Saver:
    def __init__(self, model: torch.nn.Module, sparse_optim=None, output_dir: str = "./", max_keep: int = 1, concurrency: int = 4):
        self._model = model
        self._sparse_state_dict, self._dense_state_dict = split_sparse_dense_state_dict(model.state_dict())
        self._checkpoint_file = "checkpoint"
        self._checkpoint_version_list = []
        self._max_keep = max_keep
        self._extra_save_dict = {}
        # an output_dir of the form model.<project>.<name>[/version=...] is a model-store URI: the run writes into the version's
        # directory and every checkpoint saved or removed is recorded there (``recis/framework/checkpoint_manager.py:73-78``)
        self._mos = Mos(output_dir) if str(output_dir).startswith("model.") else None
        self._output_dir = self._mos.real_physical_path if self._mos else output_dir
        self._remote = None                                   # (fsspec file system, root path) of a remote output_dir
        if _is_remote(self._output_dir):
            self._remote = _remote_fs(self._output_dir)
            self._output_dir = os.path.join(_staging_root(), "out-" + hashlib.sha1(str(output_dir).encode()).hexdigest()[:12])
            os.makedirs(self._output_dir, exist_ok=True)
        self._sparse_optim = sparse_optim
        self._concurrency = concurrency
        self._io_state = {}
        self._sparse_optim_state = {}

    def register_io_state(self, name, obj):
        if name in self._io_state:
            raise ValueError(f"name {name} already registered in io state")
        self._io_state[name] = obj

    def register_for_checkpointing(self, name, obj):
        if name in self._extra_save_dict:
            raise ValueError(f"name {name} already registered")
        self._extra_save_dict[name] = obj

    def get_extra_data(self, name: str):
        return self._extra_save_dict.get(name)

    def _sparse_parts(self):
        """(tables, scalar tensors of the sparse optimizer) as they stand now."""
        state = dict(self._sparse_state_dict)
        if self._sparse_optim is not None:
            state.update(self._sparse_optim.state_dict())
        return split_sparse_dense_state_dict(state)

    def save(self, ckpt_id: str, shard_id: int = 0, shard_num: int = 1):
        ckpt_path = os.path.join(self._output_dir, ckpt_id)
        os.makedirs(ckpt_path, exist_ok=True)
        logger.info(f"Save checkpoint {ckpt_id} to {ckpt_path}")
        tables, scalars = self._sparse_parts()
        if tables:
            self.save_sparse_params(shard_id, shard_num, ckpt_path, {**tables, **scalars}, self._concurrency)
        io_states = {name: io.dump_io_state() for name, io in self._io_state.items()}
        if io_states:
            torch.save(io_states, os.path.join(ckpt_path, f"io_state_{shard_id}.pt"))
        if shard_id == 0:
            _tables, dense = split_sparse_dense_state_dict(self._model.state_dict())
            if dense:
                self.save_dense_params(ckpt_path, dense)
            if self._extra_save_dict:
                extra = {k: (v.state_dict() if hasattr(v, "state_dict") else v) for k, v in self._extra_save_dict.items()}
                torch.save(extra, os.path.join(ckpt_path, "extra.pt"))
                if io_states:
                    with open(os.path.join(ckpt_path, "io_state_count"), "w") as f:
                        f.write(f"{shard_num}")
            listing = os.path.join(self._output_dir, self._checkpoint_file)
            known = [l.strip() for l in open(listing).read().split("\n") if l.strip()] if os.path.exists(listing) else []
            if ckpt_id not in known:          # saving the same step twice (interval save + final save) lists it once
                with open(listing, "a+") as f:
                    f.write(ckpt_id + "\n")
            if ckpt_id not in self._checkpoint_version_list:
                self._checkpoint_version_list.append(ckpt_id)
            while len(self._checkpoint_version_list) > self._max_keep:
                old = self._checkpoint_version_list.pop(0)
                logger.info(f"Remove checkpoint {os.path.join(self._output_dir, old)}")
                shutil.rmtree(os.path.join(self._output_dir, old), ignore_errors=True)
                if self._remote:
                    fs, root = self._remote
                    if fs.exists(f"{root}/{old}"):
                        fs.rm(f"{root}/{old}", recursive=True)
                with open(os.path.join(self._output_dir, self._checkpoint_file)) as f:
                    remains = [l.strip() for l in f.read().split("\n") if l.strip() and l.strip() != old]
                with open(os.path.join(self._output_dir, self._checkpoint_file), "w") as f:
                    f.writelines(r + "\n" for r in remains)
                if self._mos:
                    self._mos.ckpt_update(ckpt_id=old, path=os.path.join(self._output_dir, old), is_delete=True)
            if self._mos:
                self._mos.ckpt_update(ckpt_id=ckpt_id, path=ckpt_path)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if self._remote:
            self._upload(ckpt_id, shard_id)

    def _upload(self, ckpt_id: str, shard_id: int):
        """Copy what this rank wrote of ``ckpt_id`` to the remote directory; the listing goes last, from rank 0, once every rank
        has uploaded (a reader that sees a checkpoint listed finds all of its files)."""
        fs, root = self._remote
        local = os.path.join(self._output_dir, ckpt_id)
        for dirpath, _dirs, files in os.walk(local):
            rel = os.path.relpath(dirpath, self._output_dir)
            fs.makedirs(f"{root}/{rel}", exist_ok=True)
            for f in files:
                fs.put_file(os.path.join(dirpath, f), f"{root}/{rel}/{f}")
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        if shard_id == 0:
            fs.put_file(os.path.join(self._output_dir, self._checkpoint_file), f"{root}/{self._checkpoint_file}")

    def _download(self, fs, root: str, ckpt_id: Optional[str], local_root: str) -> Optional[str]:
        """Bring the listing and one checkpoint (the last listed when ``ckpt_id`` is None) from ``root`` into ``local_root``;
        returns the checkpoint id, or None when the remote directory lists none."""
        os.makedirs(local_root, exist_ok=True)
        listing = f"{root}/{self._checkpoint_file}"
        if ckpt_id is None:
            if not fs.exists(listing):
                return None
            fs.get_file(listing, os.path.join(local_root, self._checkpoint_file))
            lines = [l.strip() for l in open(os.path.join(local_root, self._checkpoint_file)).read().split("\n") if l.strip()]
            if not lines:
                return None
            ckpt_id = lines[-1]
        if not fs.exists(f"{root}/{ckpt_id}"):
            return None
        for dirpath, _dirs, files in fs.walk(f"{root}/{ckpt_id}"):
            # file systems differ in whether listed paths keep the leading slash: compare without it
            base, here = root.strip("/"), dirpath.strip("/")
            rel = here[len(base):].strip("/") if here.startswith(base) else ckpt_id
            os.makedirs(os.path.join(local_root, rel), exist_ok=True)
            for f in files:
                target = os.path.join(local_root, rel, f)
                if not os.path.exists(target) or os.path.getsize(target) != fs.size(f"{dirpath}/{f}"):
                    fs.get_file(f"{dirpath}/{f}", target)
        return ckpt_id

    # ---- the pieces of save(), callable on their own as in the reference (``recis/framework/checkpoint_manager.py:222-274``)
    def save_sparse_params(self, shard_id: int, shard_num: int, ckpt_path: str, sparse_state_dict: dict, concurrent: int = 16,
                           sync_func=None):
        """Write this shard's tables (and the dense tensors mixed into ``sparse_state_dict``, e.g. the sparse optimizer's scalars)
        as a safetensors bundle under ``ckpt_path``; ``sync_func`` (default: a barrier when there are several shards) runs after
        the write."""
        tables, tensors = split_sparse_dense_state_dict(dict(sparse_state_dict))
        SSaver(shard_index=shard_id, shard_num=shard_num, parallel=concurrent, hashtables=tables, tensors=tensors, path=ckpt_path).save()
        if sync_func is None:
            if shard_num > 1 and dist.is_available() and dist.is_initialized():
                dist.barrier()
        else:
            sync_func()

    def save_dense_params(self, ckpt_path: str, dense_state_dict: dict):
        torch.save(dense_state_dict, os.path.join(ckpt_path, "model.pt"))

    def save_sparse_meta(self, dirname: str):
        """Kept for API compatibility: the reference concatenates per-writer index files here; this writer merges the shards'
        metadata into ``index`` / ``tensorkey.json`` itself (a gather on the process group), so there is nothing left to do."""
        return None

    def load_sparse_optim(self):
        """Apply the sparse optimizer scalars read by the last ``load_sparse_params`` call."""
        if self._sparse_optim is not None and self._sparse_optim_state:
            logger.info("Load sparse optim")
            self._sparse_optim.load_state_dict(self._sparse_optim_state)

    # ---- loading
    def load_sparse_params(self, ckpt_dir: str, strict=True, with_optim_scalars=True):
        tables, scalars = self._sparse_parts()
        loaded = {k: v.clone() for k, v in scalars.items()} if with_optim_scalars else {}
        SLoader(ckpt_dir, hashtables=tables, tensors=loaded, strict=strict).load()
        self._sparse_optim_state = loaded
        return loaded

    def load_dense_params(self, ckpt_dir: str, strict: bool = True):
        logger.info("Load dense model")
        self._model.load_state_dict(torch.load(os.path.join(ckpt_dir, "model.pt"), weights_only=False), strict=strict)

    def load_extra_params(self, ckpt_dir: str, load_io: bool, shard_id: int = 0):
        extra = torch.load(os.path.join(ckpt_dir, "extra.pt"), weights_only=False)
        if load_io and self._io_state:
            count_file = os.path.join(ckpt_dir, "io_state_count")
            io_file = os.path.join(ckpt_dir, f"io_state_{shard_id}.pt")
            if os.path.exists(count_file) and os.path.exists(io_file):
                io_state = torch.load(io_file, weights_only=False)
                for name, io in self._io_state.items():
                    if name in io_state:
                        logger.info(f"Load io state for dataset: {name}")
                        io.load_io_state(io_state[name])
        for key, value in list(self._extra_save_dict.items()):
            if key not in extra:
                continue
            if hasattr(value, "load_state_dict"):
                value.load_state_dict(extra[key])
            elif isinstance(value, torch.Tensor) and isinstance(extra[key], torch.Tensor):
                value.copy_(extra[key])
            else:
                self._extra_save_dict[key] = extra[key]

    def load(self, ckpt_path: Optional[str] = None, ckpt_id: Optional[str] = None, load_conf: Optional[dict] = None, shard_id: int = 0,
             direct_path=False):
        load_conf = load_conf or {}
        if direct_path:
            if not ckpt_path:
                return False
            if _is_remote(ckpt_path):                       # a model bank on a remote file system: fetch it, then load locally
                fs, root = _remote_fs(ckpt_path)
                parent, name = root.rstrip("/").rsplit("/", 1)
                local_root = os.path.join(_staging_root(), "bank-" + hashlib.sha1(str(ckpt_path).encode()).hexdigest()[:12])
                if self._download(fs, parent, name, local_root) is None:
                    raise FileNotFoundError(f"no checkpoint at {ckpt_path}")
                ckpt_path = os.path.join(local_root, name)
        else:
            if ckpt_path is None and self._remote:
                fs, root = self._remote
                found = self._download(fs, root, ckpt_id, self._output_dir)
                if found is None:
                    logger.info(f"Checkpoint not found in {root}")
                    return False
                ckpt_id = found
            ckpt_path = ckpt_path or self._output_dir
            if ckpt_id is None:
                listing = os.path.join(ckpt_path, self._checkpoint_file)
                if not os.path.exists(listing):
                    logger.info(f"Checkpoint not found in {ckpt_path}")
                    return False
                lines = [l.strip() for l in open(listing).read().split("\n") if l.strip()]
                if not lines:
                    return False
                ckpt_id = lines[-1]
            ckpt_path = os.path.join(ckpt_path, ckpt_id)
        logger.info(f"Load checkpoint conf {load_conf} from {ckpt_path}")
        self.load_by_config(ckpt_path, load_conf, shard_id)
        return True

    def load_by_config(self, ckpt_path: str, load_conf: Optional[dict] = None, shard_id: int = 0):
        load_conf = load_conf or {}
        parts = ["sparse", "dense", "extra", "sparse_opt", "io_state"]
        load_map = dict.fromkeys(parts, False)
        for item in load_conf.get("load", ["*"]):
            for p in (parts if item == "*" else [item]):
                load_map[p] = True
        for item in load_conf.get("exclude", []):
            for p in (parts if item == "*" else [item]):
                load_map[p] = False
        strict = load_conf.get("strict", True)
        scalars = {}
        if load_map["sparse"] and self._sparse_state_dict:
            scalars = self.load_sparse_params(ckpt_path, strict=strict, with_optim_scalars=load_map["sparse_opt"])
        if load_map["dense"] and self._dense_state_dict and os.path.exists(os.path.join(ckpt_path, "model.pt")):
            self.load_dense_params(ckpt_path, strict=strict)
        if load_map["extra"] and self._extra_save_dict and os.path.exists(os.path.join(ckpt_path, "extra.pt")):
            self.load_extra_params(ckpt_path, load_map["io_state"], shard_id)
        if load_map["sparse_opt"] and scalars:
            self.load_sparse_optim()


class CheckpointManager:
    def __init__(self, saver: Saver, save_interval: int) -> None:
        self._saver = saver
        self._global_step = torch.scalar_tensor(0, dtype=torch.int64)
        self._rank = int(os.environ.get("RANK", 0))
        self._shard_num = int(os.environ.get("WORLD_SIZE", 1))
        self._save_interval = save_interval
        if self._saver.get_extra_data("global_step") is None:
            self._saver.register_for_checkpointing("global_step", self._global_step)

    @property
    def save_interval(self):
        return self._save_interval

    @property
    def global_step(self):
        return self._global_step

    def register_for_checkpointing(self, name, obj):
        self._saver.register_for_checkpointing(name, obj)

    def step(self):
        self._global_step += 1
        if self._save_interval and int(self._global_step) % self._save_interval == 0:
            self.save()

    def save(self):
        """Save the current step unless it has just been saved (the final save of a run whose last step hit the interval)."""
        step = int(self._global_step)
        if getattr(self, "_last_saved_step", None) == step:
            return
        self._saver.save(f"ckpt_{step}", self._rank, self._shard_num)
        self._last_saved_step = step

    def load_model_bank(self, model_bank_conf):
        for mbc in model_bank_conf or []:
            path = mbc["path"]
            if path is not None and str(path).startswith("model."):      # a model-store URI names the checkpoint
                path = Mos(path, True).real_physical_path
            self._saver.load(ckpt_path=path, load_conf=mbc, shard_id=self._rank, direct_path=True)

    def restore(self, global_step: Optional[int] = None):
        self._saver.load(ckpt_id=None if global_step is None else f"ckpt_{global_step}", shard_id=self._rank)
        gs = self._saver.get_extra_data("global_step")
        if gs is not None:
            self._global_step = gs if isinstance(gs, torch.Tensor) else torch.scalar_tensor(int(gs), dtype=torch.int64)
        return self._global_step
