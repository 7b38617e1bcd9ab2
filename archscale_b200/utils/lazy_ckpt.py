"""Checkpoint IO that never holds a whole model in host memory twice.

Role of ``lazy_load`` / ``incremental_save`` in the reference (`lit_gpt/utils.py:101-237,302-411`), used by its
converters and evaluation scripts to stream multi-GB checkpoints:

* :class:`lazy_load` opens a ``torch.save`` file and hands out its object tree with every tensor memory-mapped from the
  file (``torch.load(mmap=True)``): a tensor's bytes are read when it is touched, tensors that are never touched
  (optimizer state, when only weights are wanted) cost nothing.  The reference re-implements the unpickler with
  ``NotYetLoadedTensor`` proxies because it predates ``mmap``.
* :class:`incremental_save` writes a file that ``torch.load`` reads, but lets the caller hand tensors over one at a time
  (:meth:`incremental_save.store_early`): their bytes go to the file immediately and the caller can drop them; the final
  :meth:`incremental_save.save` pickles the object tree, in which early-stored tensors are small placeholders.
"""
from __future__ import annotations

import pickle
import warnings
from collections import OrderedDict
from io import BytesIO
from typing import Any

import torch


class lazy_load:
    """``with lazy_load(path) as sd: w = sd["model"]["lm_head.weight"]`` — tensors are views of the mapped file."""

    def __init__(self, path, weights_only: bool = False) -> None:
        self.path = str(path)
        self.weights_only = weights_only
        self.sd = None

    def __enter__(self):
        try:
            self.sd = torch.load(self.path, map_location="cpu", mmap=True, weights_only=self.weights_only)
        except (RuntimeError, ValueError):
            # legacy (non-zip) files cannot be mapped: read them whole
            self.sd = torch.load(self.path, map_location="cpu", weights_only=self.weights_only)
        return self.sd

    def __exit__(self, *exc) -> None:
        self.sd = None


class _StoredTensor:
    """Placeholder of a tensor whose bytes are already in the file."""

    def __init__(self, key: int, storage_type, numel: int, size, stride, requires_grad: bool) -> None:
        self.key, self.storage_type, self.numel = key, storage_type, numel
        self.size, self.stride, self.requires_grad = tuple(size), tuple(stride), requires_grad

    @property
    def shape(self):
        return torch.Size(self.size)


class _StorageRef:
    def __init__(self, st: _StoredTensor) -> None:
        self.st = st


class _Pickler(pickle.Pickler):
    def __init__(self, saver: "incremental_save", buf) -> None:
        super().__init__(buf, protocol=2)
        self.saver = saver

    def persistent_id(self, obj: Any):
        if isinstance(obj, _StorageRef):
            st = obj.st
            return ("storage", st.storage_type, str(st.key), "cpu", st.numel)
        return None

    def reducer_override(self, obj: Any):
        if isinstance(obj, torch.Tensor) and not isinstance(obj, torch.nn.Parameter):
            obj = self.saver.store_early(obj)
        elif isinstance(obj, torch.nn.Parameter):
            obj = self.saver.store_early(obj.detach())
        if isinstance(obj, _StoredTensor):
            return (torch._utils._rebuild_tensor_v2, (_StorageRef(obj), 0, obj.size, obj.stride, obj.requires_grad, OrderedDict()))
        return NotImplemented


class incremental_save:
    def __init__(self, path) -> None:
        self.path = str(path)
        self.zip = torch._C.PyTorchFileWriter(self.path)
        self.next_key = 0
        self.saved = False

    def __enter__(self) -> "incremental_save":
        return self

    def store_early(self, tensor: torch.Tensor) -> _StoredTensor:
        """Write the tensor's bytes now; keep the returned placeholder in the object tree instead of the tensor."""
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"can only store tensors early, not {type(tensor)}")
        if self.saved:
            raise RuntimeError("the object tree has already been saved")
        t = tensor.detach().to("cpu").contiguous()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            storage_type = getattr(torch, t._typed_storage()._pickle_storage_type())
        key = self.next_key
        self.next_key += 1
        # the record holds exactly this tensor (a view of a larger storage is compacted by .contiguous() above)
        flat = t.reshape(-1)
        nbytes = flat.numel() * flat.element_size()
        if flat.storage_offset() != 0 or flat.untyped_storage().nbytes() != nbytes:
            flat = flat.clone()
        if nbytes == 0:
            self.zip.write_record(f"data/{key}", b"", 0)
        else:
            self.zip.write_record(f"data/{key}", flat.untyped_storage(), nbytes)
        return _StoredTensor(key, storage_type, flat.numel(), t.shape, t.stride(), False)

    def save(self, obj: Any) -> None:
        if self.saved:
            raise RuntimeError("the object tree has already been saved")
        buf = BytesIO()
        _Pickler(self, buf).dump(obj)
        data = buf.getvalue()
        self.zip.write_record("data.pkl", data, len(data))
        self.zip.write_record("byteorder", b"little", 6)
        self.saved = True

    def __exit__(self, *exc) -> None:
        self.zip.write_end_of_file()
