"""Reader for NVFP4 recipe-v2 parameters stored as SafeTensors records.

A logical NVFP4 parameter ``<name>`` is three physical records, ``<name>.payload`` (U8
``[..., ceil(K/2)]``), ``<name>.block_scales`` (U8 ``[..., ceil(K/16)]``) and
``<name>.global_scale`` (F32 scalar), as the reference's converter writes them
(tools/nvfp4/convert.py:317-319, file metadata ``nml_recipe = nml-nvfp4-weight-v2`` :331-335)
and its checkpoint crate resolves them (crates/nml-checkpoint/src/lib.rs:569-620: a base with
only some of its components present is rejected, shapes must match the logical shape).

Records may be spread over several files listed in a ``*.safetensors.index.json`` weight map.
``load_rows`` reads only the byte span of rows ``[start, stop)`` of axis 0, which is how an
expert-parallel rank takes its experts and a column-sharded head its vocabulary rows
(crates/nml-parameter/src/lib.rs:285-312: shards cut on axis 0 never split a 16-block).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from .ops import NvFp4Parameter

RECIPE = "nml-nvfp4-weight-v2"
COMPONENTS = ("payload", "block_scales", "global_scale")


class CheckpointError(ValueError):
    pass


class NvFp4Checkpoint:
    """Index of the records of one checkpoint directory (or single ``.safetensors`` file)."""

    def __init__(self, path):
        path = Path(path)
        self._files: dict[str, Path] = {}   # record name -> file
        self._recipes: dict[Path, str | None] = {}
        if path.is_dir():
            indexes = sorted(path.glob("*.safetensors.index.json"))
            if indexes:
                weight_map = json.loads(indexes[0].read_text())["weight_map"]
                for name, file in weight_map.items():
                    self._files[name] = path / file
                files = sorted(set(self._files.values()))
            else:
                files = sorted(path.glob("*.safetensors"))
                self._scan(files)
        else:
            files = [path]
            self._scan(files)
        if not files:
            raise CheckpointError(f"no SafeTensors records under {path}")
        for file in files:
            with safe_open(str(file), framework="pt", device="cpu") as handle:
                metadata = handle.metadata() or {}
                self._recipes[file] = metadata.get("nml_recipe")
                if not self._files or file not in set(self._files.values()):
                    for name in handle.keys():
                        self._files.setdefault(name, file)

    def _scan(self, files):
        for file in files:
            with safe_open(str(file), framework="pt", device="cpu") as handle:
                for name in handle.keys():
                    if name in self._files:
                        raise CheckpointError(f"record {name} appears in more than one file")
                    self._files[name] = file

    def names(self):
        return sorted(self._files)

    def nvfp4_bases(self):
        """Logical names that own all three NVFP4 components."""
        bases = {name.rsplit(".", 1)[0] for name in self._files
                 if name.rsplit(".", 1)[-1] in COMPONENTS}
        return sorted(base for base in bases if self._present(base) == len(COMPONENTS))

    def _present(self, base: str) -> int:
        return sum(f"{base}.{component}" in self._files for component in COMPONENTS)

    def _resolve(self, name: str, aliases=()) -> str:
        complete = []
        for base in (name, *aliases):
            present = self._present(base)
            if present == len(COMPONENTS):
                complete.append(base)
            elif present != 0:
                raise CheckpointError(f"NVFP4 parameter {base} has only {present} of its "
                                      f"{len(COMPONENTS)} records")
        if not complete:
            raise CheckpointError(f"missing tensor {name}")
        if len(complete) > 1:
            raise CheckpointError(f"ambiguous aliases for {name}: {complete}")
        return complete[0]

    def _slice(self, record: str):
        file = self._files[record]
        handle = safe_open(str(file), framework="pt", device="cpu")
        return handle, handle.get_slice(record)

    def load_rows(self, name: str, logical_shape, dtype: torch.dtype, start: int, stop: int,
                  device="cpu", aliases=()) -> NvFp4Parameter:
        """Rows [start, stop) of axis 0 of the logical parameter, reading only their bytes."""
        logical_shape = tuple(int(d) for d in logical_shape)
        if not logical_shape or not 0 <= start < stop <= logical_shape[0]:
            raise CheckpointError(f"row range [{start}, {stop}) outside {logical_shape}")
        base = self._resolve(name, aliases)
        width = logical_shape[-1]
        expected = {"payload": logical_shape[:-1] + ((width + 1) // 2,),
                    "block_scales": logical_shape[:-1] + ((width + 15) // 16,)}
        parts = {}
        for component, shape in expected.items():
            record = f"{base}.{component}"
            handle, view = self._slice(record)
            with handle:
                if view.get_dtype() != "U8":
                    raise CheckpointError(f"{record} must be U8, found {view.get_dtype()}")
                if tuple(view.get_shape()) != shape:
                    raise CheckpointError(f"{record}: expected shape {shape}, found "
                                          f"{tuple(view.get_shape())}")
                parts[component] = view[start:stop]
        record = f"{base}.global_scale"
        handle, view = self._slice(record)
        with handle:
            if view.get_dtype() != "F32" or tuple(view.get_shape()) not in ((), (1,)):
                raise CheckpointError(f"{record} must be an F32 scalar")
            global_scale = view[:] if view.get_shape() else handle.get_tensor(record)
        recipe = self._recipes.get(self._files[f"{base}.payload"])
        if recipe is not None and recipe != RECIPE:
            raise CheckpointError(f"{base}: recipe {recipe!r}, this reader takes {RECIPE!r}")
        shape = (stop - start,) + logical_shape[1:]
        return NvFp4Parameter.nvfp4(
            name, shape, dtype, parts["payload"].to(device), parts["block_scales"].to(device),
            global_scale.reshape(()).to(torch.float32).to(device))

    def load(self, name: str, logical_shape, dtype: torch.dtype, device="cpu",
             aliases=()) -> NvFp4Parameter:
        return self.load_rows(name, logical_shape, dtype, 0, int(logical_shape[0]), device,
                              aliases)

    def load_shard(self, name: str, logical_shape, dtype: torch.dtype, rank: int, world: int,
                   device="cpu", aliases=()) -> NvFp4Parameter:
        """The contiguous axis-0 shard of ``rank`` (experts of an expert-parallel rank, rows of
        a column-sharded head; crates/nml-sharding/src/lib.rs:180-213)."""
        extent = int(logical_shape[0])
        if extent % world != 0:
            raise CheckpointError(f"axis extent {extent} does not divide evenly over {world}")
        length = extent // world
        return self.load_rows(name, logical_shape, dtype, rank * length, (rank + 1) * length,
                              device, aliases)

    def load_dense(self, name: str, device="cpu") -> torch.Tensor:
        if name not in self._files:
            raise CheckpointError(f"missing tensor {name}")
        with safe_open(str(self._files[name]), framework="pt", device="cpu") as handle:
            return handle.get_tensor(name).to(device)


def save_nvfp4(path, parameters: dict, dense: dict | None = None) -> None:
    """Writes logical NVFP4 parameters (and dense tensors) as recipe-v2 records, the layout of
    the reference's converter (tools/nvfp4/convert.py:296-339)."""
    from safetensors.torch import save_file
    records = {}
    for name, parameter in parameters.items():
        records[f"{name}.payload"] = parameter.payload.cpu().contiguous()
        records[f"{name}.block_scales"] = parameter.block_scales.cpu().contiguous()
        records[f"{name}.global_scale"] = parameter.global_scale.cpu().reshape(()).contiguous()
    for name, tensor in (dense or {}).items():
        records[name] = tensor.cpu().contiguous()
    save_file(records, str(path), metadata={"format": "pt", "nml_recipe": RECIPE})
