"""The file side of the weight loader: safetensors shards through mmap, the checkpoint index, the
tensor names of the model and the check against the architecture (crates/qwc-model/src/safetensors.rs,
checkpoint.rs, names.rs; the loop of crates/qwc-engine/src/weights.rs:200-360 that walks the layers and
drops file pages behind it).

A shard is `[8-byte little-endian header length][JSON header][data]`; offsets in the header count from
the start of the data block.  Tensors are handed out as views of the mapping - nothing is copied until
`weights.py` reshapes a projection for the engine.  `write_shard` / `write_checkpoint` produce the same
format, for tests and for exporting an engine's tensors.

The engine is specialised for one architecture, so a shape that differs is a load error, not a reason
to adapt (checkpoint.rs:1-5).  The architecture here is the engine's config: the layer widths follow
from it the way crates/qwc-core/src/arch.rs derives them from its constants.
"""

from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np

from . import weights

EMBED = "model.language_model.embed_tokens.weight"
FINAL_NORM = "model.language_model.norm.weight"
LM_HEAD = "lm_head.weight"

# safetensors dtype -> (bytes per element, numpy view)
DTYPES = {"BF16": (2, np.uint16), "F32": (4, np.float32), "F8_E4M3": (1, np.uint8), "U8": (1, np.uint8)}
QUANT_SUFFIXES = ("weight_packed", "weight_scale", "weight_global_scale", "input_global_scale")


class CheckpointError(ValueError):
    """A shard or an index that does not parse, or a tensor that is not what the architecture says."""


def layer_prefix(index: int) -> str:
    return f"model.language_model.layers.{index}"


def _block(config, layer: int) -> str:
    return "self_attn" if (layer + 1) % config.full_attention_interval == 0 else "linear_attn"


def quant_linears(config, layer: int) -> list:
    """(tensor prefix, short name, out_features, in_features) of every quantised projection of a layer
    (names.rs:14-59)."""
    prefix, block = layer_prefix(layer), _block(config, layer)
    out = []
    for name, (rows, cols) in weights.layer_shapes(config, layer).items():
        owner = "mlp" if name in ("gate_proj", "up_proj", "down_proj") else block
        out.append((f"{prefix}.{owner}.{name}", name, rows, cols))
    return out


def plain_tensors(config, layer: int) -> list:
    """(tensor name, short name, shape) of the unquantised tensors of a layer (names.rs:61-91)."""
    prefix = layer_prefix(layer)
    heads = config.delta_value_heads
    channels = 2 * 16 * 128 + heads * 128
    shapes = {"input_layernorm.weight": [config.hidden], "post_attention_layernorm.weight": [config.hidden],
              "self_attn.q_norm.weight": [256], "self_attn.k_norm.weight": [256],
              "linear_attn.conv1d.weight": [channels, 1, 4], "linear_attn.A_log": [heads],
              "linear_attn.dt_bias": [heads], "linear_attn.norm.weight": [128]}
    return [(f"{prefix}.{short}", short, shapes[short]) for short in weights.plain_names(config, layer)]


class TensorInfo:
    def __init__(self, dtype: str, shape, start: int, end: int):
        self.dtype, self.shape, self.start, self.end = dtype, list(shape), start, end

    def elems(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

    def bytes(self) -> int:
        return self.end - self.start


class Shard:
    """One safetensors file, mapped read-only (safetensors.rs:66-150)."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as file:
            size = os.fstat(file.fileno()).st_size
            if size < 8:
                raise CheckpointError(f"{path}: shard shorter than its header length")
            self._map = mmap.mmap(file.fileno(), 0, access=mmap.ACCESS_READ)
        if hasattr(mmap, "MADV_SEQUENTIAL"):
            self._map.madvise(mmap.MADV_SEQUENTIAL)
        (header_length,) = struct.unpack("<Q", self._map[:8])
        self.data_offset = 8 + header_length
        if self.data_offset > size:
            raise CheckpointError(f"{path}: header length goes past the end of the file")
        try:
            header = json.loads(bytes(self._map[8:self.data_offset]))
        except ValueError as error:
            raise CheckpointError(f"{path}: header does not parse: {error}") from None
        if not isinstance(header, dict):
            raise CheckpointError(f"{path}: header is not an object")
        self._bytes = np.frombuffer(self._map, dtype=np.uint8)
        self.tensors = {}
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (start, end) = entry["dtype"], entry["shape"], entry["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise CheckpointError(f"{path}: {name}: no dtype, shape or data_offsets") from None
            if dtype not in DTYPES:
                raise CheckpointError(f"{path}: unsupported type {dtype} for {name}")
            info = TensorInfo(dtype, shape, int(start), int(end))
            if info.start > info.end or self.data_offset + info.end > size:
                raise CheckpointError(f"{path}: {name}: data outside the file")
            if info.bytes() != info.elems() * DTYPES[dtype][0]:
                raise CheckpointError(f"{path}: {name}: {info.bytes()} bytes for shape {info.shape} of {dtype}")
            self.tensors[name] = info

    def info(self, name: str):
        return self.tensors.get(name)

    def bytes(self, name: str):
        """Raw bytes of a tensor: a view of the mapping, no copy."""
        info = self.tensors.get(name)
        if info is None:
            return None
        return self._bytes[self.data_offset + info.start:self.data_offset + info.end]

    def names(self):
        return self.tensors.keys()

    def evict_pages(self) -> None:
        """Drops the clean file pages behind tensors that have been uploaded; the mapping stays valid and
        pages fault in again on the next access (safetensors.rs:140-150)."""
        if hasattr(mmap, "MADV_DONTNEED"):
            self._map.madvise(mmap.MADV_DONTNEED)


class Checkpoint:
    """A directory with `model.safetensors.index.json` and its shards (checkpoint.rs:56-110)."""

    def __init__(self, directory: str):
        index_path = os.path.join(directory, "model.safetensors.index.json")
        try:
            with open(index_path, "rb") as file:
                index = json.load(file)
        except ValueError as error:
            raise CheckpointError(f"{index_path}: does not parse: {error}") from None
        weight_map = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(weight_map, dict):
            raise CheckpointError("index has no weight_map")
        files = sorted({file for file in weight_map.values() if isinstance(file, str)})
        self.shards = [Shard(os.path.join(directory, file)) for file in files]
        position = {file: i for i, file in enumerate(files)}
        self.location = {name: position[file] for name, file in weight_map.items() if file in position}

    @classmethod
    def open(cls, directory: str) -> "Checkpoint":
        return cls(directory)

    def info(self, name: str):
        shard = self.location.get(name)
        return None if shard is None else self.shards[shard].info(name)

    def bytes(self, name: str):
        shard = self.location.get(name)
        return None if shard is None else self.shards[shard].bytes(name)

    def array(self, name: str):
        """The tensor as a numpy view in its own element type and shape (bf16 as uint16 bit patterns)."""
        info, raw = self.info(name), self.bytes(name)
        if info is None or raw is None:
            return None
        return raw.view(DTYPES[info.dtype][1]).reshape(info.shape)

    def scalar_f32(self, name: str):
        raw = self.bytes(name)
        if raw is None or raw.size < 4:
            return None
        return float(raw[:4].view(np.float32)[0])

    def tensor_count(self) -> int:
        return len(self.location)

    def quant_linear(self, prefix: str, out_features: int, in_features: int) -> weights.QuantLinear:
        """A quantised projection by prefix, checked against the architecture (checkpoint.rs:112-172)."""
        packed_name, scale_name = f"{prefix}.weight_packed", f"{prefix}.weight_scale"
        for name, shape, dtype in ((packed_name, [out_features, in_features // 2], "U8"),
                                   (scale_name, [out_features, in_features // 16], "F8_E4M3")):
            info = self.info(name)
            if info is None:
                raise CheckpointError(f"missing {name}")
            if info.shape != shape:
                raise CheckpointError(f"{name}: shape {info.shape}, expected {shape}")
            if info.dtype != dtype:
                raise CheckpointError(f"{name}: type {info.dtype}, expected {dtype}")
        scales = {}
        for which in ("weight_global_scale", "input_global_scale"):
            scales[which] = self.scalar_f32(f"{prefix}.{which}")
            if scales[which] is None:
                raise CheckpointError(f"missing {prefix}.{which}")
        linear = weights.QuantLinear(self.array(packed_name), self.array(scale_name), scales["weight_global_scale"])
        linear.input_global_scale = scales["input_global_scale"]  # W4A4 only: the W4A16 path does not read it
        return linear

    def validate(self, config) -> tuple:
        """Full check against the architecture: (list of mismatches, statistics) (checkpoint.rs:174-262).
        The draft head's tensors (`mtp.*`) are counted when present and not asked for: this engine does
        not run it."""
        problems = []
        stats = {"tensors": 0, "quantized_linears": 0, "packed_bytes": 0, "scale_bytes": 0, "plain_bytes": 0,
                 "embed_bytes": 0, "lm_head_bytes": 0, "mtp_bytes": 0, "unused_bytes": 0, "unused_tensors": 0}
        seen = set()

        def check_plain(name, shape, field="plain_bytes"):
            seen.add(name)
            info = self.info(name)
            if info is None:
                problems.append(f"missing {name}")
                return
            if info.shape != list(shape):
                problems.append(f"{name}: shape {info.shape}, expected {list(shape)}")
            stats[field] += info.bytes()
            stats["tensors"] += 1

        check_plain(FINAL_NORM, [config.hidden])
        check_plain(EMBED, [config.vocab, config.hidden], "embed_bytes")
        check_plain(LM_HEAD, [config.vocab, config.hidden], "lm_head_bytes")
        for layer in range(config.num_layers):
            for name, _, shape in plain_tensors(config, layer):
                check_plain(name, shape)
            for prefix, _, rows, cols in quant_linears(config, layer):
                try:
                    linear = self.quant_linear(prefix, rows, cols)
                    stats["quantized_linears"] += 1
                    stats["packed_bytes"] += linear.packed.nbytes
                    stats["scale_bytes"] += linear.block_scales.nbytes
                    stats["tensors"] += 4
                except (CheckpointError, weights.LoadError) as error:
                    problems.append(str(error))
                seen.update(f"{prefix}.{suffix}" for suffix in QUANT_SUFFIXES)
        for name in self.location:
            if name in seen:
                continue
            info = self.info(name)
            if info is None:
                continue
            if name.startswith("mtp."):
                stats["mtp_bytes"] += info.bytes()
                stats["tensors"] += 1
            else:
                stats["unused_bytes"] += info.bytes()
                stats["unused_tensors"] += 1
        return problems, stats

    def evict_file_pages(self) -> None:
        """Releases the mapped pages from the process's working set; a loader calls this between upload
        phases to keep to a small host-memory envelope (checkpoint.rs:264-271)."""
        for shard in self.shards:
            shard.evict_pages()

    # ---- the loader's walk over the model ----
    def layer(self, config, layer: int) -> tuple:
        """(projections, plain) of one layer in the form `weights.load_layer` takes."""
        projections = {short: self.quant_linear(prefix, rows, cols)
                       for prefix, short, rows, cols in quant_linears(config, layer)}
        plain = {}
        for name, short, shape in plain_tensors(config, layer):
            info = self.info(name)
            if info is None:
                raise CheckpointError(f"missing {name}")
            if info.shape != list(shape) or info.dtype != "BF16":
                raise CheckpointError(f"{name}: {info.dtype} {info.shape}, expected BF16 {list(shape)}")
            plain[short] = self.array(name).reshape(-1)
        return projections, plain

    def vocab_table(self, config, name: str):
        info = self.info(name)
        if info is None:
            raise CheckpointError(f"missing {name}")
        if info.shape != [config.vocab, config.hidden] or info.dtype != "BF16":
            raise CheckpointError(f"{name}: {info.dtype} {info.shape}, expected BF16 {[config.vocab, config.hidden]}")
        return self.array(name)


def load(engine, checkpoint: Checkpoint, evict: bool = True) -> dict:
    """The whole model into an engine, layer by layer, dropping the file pages of what has been uploaded
    (weights.rs:200-360).  Returns the byte counts of `weights.load_model`."""
    config = engine.config
    problems, _ = checkpoint.validate(config)
    if problems:
        raise CheckpointError("; ".join(problems[:8]) + (f" (+{len(problems) - 8} more)" if len(problems) > 8 else ""))
    total = {"quantized_bytes": 0, "projections": 0, "plain_bytes": 0, "vocab_bytes": 0}
    for layer in range(config.num_layers):
        projections, plain = checkpoint.layer(config, layer)
        for key, value in weights.load_layer(engine, layer, projections, plain).items():
            total[key] += value
        del projections, plain
        if evict:
            checkpoint.evict_file_pages()
    norm = checkpoint.array(FINAL_NORM).reshape(-1)
    engine.write("final_norm", 0, np.ascontiguousarray(norm))
    total["plain_bytes"] += norm.nbytes
    for name, tensor in (("embed", EMBED), ("lm_head", LM_HEAD)):
        total["vocab_bytes"] += weights.load_vocab(engine, name, checkpoint.vocab_table(config, tensor))
        if evict:
            checkpoint.evict_file_pages()
    return total


# ---- writing the format (tests; exporting an engine's tensors) ----
def _raw(array: np.ndarray) -> tuple:
    """(safetensors dtype, shape, bytes) of a numpy array; uint16 arrays are bf16 bit patterns."""
    kinds = {np.dtype(np.uint16): "BF16", np.dtype(np.float32): "F32", np.dtype(np.uint8): "U8"}
    array = np.ascontiguousarray(array)
    if array.dtype not in kinds:
        raise CheckpointError(f"no safetensors type for {array.dtype}")
    return kinds[array.dtype], list(array.shape), array.tobytes()


def write_shard(path: str, tensors: dict, dtypes: dict | None = None) -> None:
    """Writes `name -> numpy array` as one safetensors file.  `dtypes[name]` overrides the type tag of a
    uint8 array ("F8_E4M3" for block scales)."""
    header, blobs, offset = {}, [], 0
    for name, array in tensors.items():
        dtype, shape, raw = _raw(array)
        dtype = (dtypes or {}).get(name, dtype)
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode()
    encoded += b" " * (-len(encoded) % 8)  # the data block starts on an 8-byte boundary
    with open(path, "wb") as file:
        file.write(struct.pack("<Q", len(encoded)))
        file.write(encoded)
        for raw in blobs:
            file.write(raw)


def write_checkpoint(directory: str, tensors: dict, dtypes: dict | None = None, tensors_per_shard: int = 64) -> None:
    """Splits `tensors` over shards of `tensors_per_shard` tensors and writes the index beside them."""
    os.makedirs(directory, exist_ok=True)
    names = list(tensors)
    count = max(1, -(-len(names) // tensors_per_shard))
    weight_map = {}
    for shard in range(count):
        file = f"model-{shard + 1:05d}-of-{count:05d}.safetensors"
        chunk = names[shard * tensors_per_shard:(shard + 1) * tensors_per_shard]
        write_shard(os.path.join(directory, file), {name: tensors[name] for name in chunk}, dtypes)
        weight_map.update({name: file for name in chunk})
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as file:
        json.dump({"metadata": {}, "weight_map": weight_map}, file)


def checkpoint_tensors(config, layers, final_norm, embed_bf16, lm_head_bf16) -> tuple:
    """`name -> array` (and the dtype overrides) of a model given in the loader's form
    (`layers[i] = (projections, plain)` as `weights.load_layer` takes them): the inverse of
    `Checkpoint.layer`, for writing a checkpoint."""
    tensors, dtypes = {}, {}
    for layer, (projections, plain) in enumerate(layers):
        for prefix, short, _, _ in quant_linears(config, layer):
            linear = projections[short]
            tensors[f"{prefix}.weight_packed"] = linear.packed
            tensors[f"{prefix}.weight_scale"] = linear.block_scales
            dtypes[f"{prefix}.weight_scale"] = "F8_E4M3"
            tensors[f"{prefix}.weight_global_scale"] = np.array([linear.weight_global_scale], dtype=np.float32)
            tensors[f"{prefix}.input_global_scale"] = np.array(
                [getattr(linear, "input_global_scale", 1.0)], dtype=np.float32)
        for name, short, shape in plain_tensors(config, layer):
            tensors[name] = np.ascontiguousarray(plain[short], dtype=np.uint16).reshape(shape)
    tensors[FINAL_NORM] = np.ascontiguousarray(final_norm, dtype=np.uint16).reshape(-1)
    tensors[EMBED] = np.ascontiguousarray(embed_bf16, dtype=np.uint16)
    tensors[LM_HEAD] = np.ascontiguousarray(lm_head_bf16, dtype=np.uint16)
    return tensors, dtypes
