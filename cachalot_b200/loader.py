"""Expert bank loader: routed experts of a checkpoint directory (safetensors shards) into a `SlabBank` in HBM.

Two on-disk layouts, as the reference reads them (storage/index.py:79-193, storage/reader.py:182-260):
  * the shipped FP4 checkpoint: one tensor per expert and field, `layers.<L>.ffn.experts.<E>.w{1,2,3}.{weight,scale}`
    (E2M1 nibbles uint8 [N, K/2], E8M0 bytes uint8 [N, K/32]);
  * a converted affine bank: every layer's experts stacked per projection field,
    `language_model.layers.<L>.ffn.experts.w{1,2,3}.{weight,scales,biases}` with shape [n_experts, rows, cols]
    (uint32 words, f16 or bf16 scales and biases; bits and group size come from `config.json`,
    benchmarks/build_affine_bank.py:72-187).
The byte ranges of an expert are read with preadv straight into a pinned staging record laid out like a bank slot
and copied to the slot with one asynchronous copy; two staging records alternate, so the read of expert i+1 runs
under the copy of expert i.  Nothing is converted on the way: a slot holds the file's bytes.
"""
from __future__ import annotations

import json
import os
import re
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

from .bank import FP4_FORMAT, ExpertFormat, SlabBank

_PER_EXPERT = re.compile(r"^layers\.(\d+)\.ffn\.experts\.(\d+)\.(w[123])\.(weight|scale)$")
_STACKED = re.compile(r"^language_model\.layers\.(\d+)\.ffn\.experts\.(w[123])\.(weight|scales|biases)$")
_ITEM = {"U32": (4, "uint32"), "F32": (4, "float32"), "F16": (2, "float16"), "BF16": (2, "bfloat16"), "U8": (1, "uint8")}


@dataclass(frozen=True)
class TensorRange:
    """Bytes [start, end) of `shard` that hold tensor `name` (short name = its last two dotted parts)."""

    name: str
    shard: Path
    start: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.start

    @property
    def short(self) -> str:
        return ".".join(self.name.rsplit(".", 2)[-2:])


@dataclass(frozen=True)
class ExpertEntry:
    layer: int
    expert: int
    tensors: tuple[TensorRange, ...]


def read_safetensors_header(path: Path) -> tuple[dict, int]:
    """(header dict, offset of the data section) of one safetensors file."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return header, 8 + n


def _shards(root: Path):
    for shard in sorted(root.glob("model-*.safetensors")):
        try:
            yield shard, *read_safetensors_header(shard)
        except (OSError, json.JSONDecodeError, struct.error):
            continue   # a shard that is still being written: index what is there


def _finish(found: dict) -> dict[tuple[int, int], ExpertEntry]:
    return {key: ExpertEntry(key[0], key[1], tuple(sorted(ranges, key=lambda r: (str(r.shard), r.start)))) for key, ranges in found.items()}


def build_expert_index(model_path) -> dict[tuple[int, int], ExpertEntry]:
    """(layer, expert) -> byte ranges of the six FP4 tensors (storage/index.py:79-121)."""
    found: dict = {}
    for shard, header, base in _shards(Path(model_path)):
        for name, meta in header.items():
            m = _PER_EXPERT.match(name)
            if m:
                lo, hi = meta["data_offsets"]
                found.setdefault((int(m.group(1)), int(m.group(2))), []).append(TensorRange(name, shard, base + lo, base + hi))
    return _finish(found)


def build_stacked_expert_index(model_path, quantized_modules: dict) -> tuple[ExpertFormat, dict[tuple[int, int], ExpertEntry]]:
    """Format and index of a converted affine bank whose experts are stacked per layer (storage/index.py:124-179)."""
    found: dict = {}
    shapes: dict = {}
    dtypes: dict = {}
    quant = None
    for shard, header, base in _shards(Path(model_path)):
        for name, meta in header.items():
            m = _STACKED.match(name)
            if not m:
                continue
            layer, proj, field = int(m.group(1)), m.group(2), m.group(3)
            spec = quantized_modules.get(f"language_model.layers.{layer}.ffn.experts.{proj}")
            if spec is None or spec.get("mode") != "affine":
                raise ValueError(f"{name}: routed experts must be affine-quantized, got {spec}")
            this = (int(spec["bits"]), int(spec.get("group_size", 64)))
            if quant is None:
                quant = this
            elif this != quant:
                raise ValueError(f"{name}: mixed expert quantization ({spec} vs {quant[0]}-bit/{quant[1]})")
            n_experts, rows, cols = (int(v) for v in meta["shape"])
            short = f"{proj}.{field}"
            if shapes.setdefault(short, (rows, cols)) != (rows, cols):
                raise ValueError(f"{name}: shape {(rows, cols)} differs from {shapes[short]}")
            item, dtypes[short] = _ITEM[meta["dtype"]]
            per = rows * cols * item
            first = base + meta["data_offsets"][0]
            for e in range(n_experts):
                found.setdefault((layer, e), []).append(
                    TensorRange(f"layers.{layer}.ffn.experts.{e}.{short}", shard, first + e * per, first + (e + 1) * per))
    if quant is None:
        raise ValueError(f"no stacked routed-expert tensors under {model_path}")
    from .bank import TENSOR_NAMES_AFFINE

    lacking = [n for n in TENSOR_NAMES_AFFINE if n not in shapes]
    if lacking:
        raise ValueError(f"stacked bank under {model_path} lacks {lacking}")
    # the kernels take a record's tensors in this fixed order (weight, scales, biases per projection)
    fmt = ExpertFormat(kind="affine", bits=quant[0], group_size=quant[1], tensor_names=TENSOR_NAMES_AFFINE, shapes=shapes, dtypes=dtypes)
    return fmt, _finish(found)


def detect_expert_bank(model_path) -> tuple[ExpertFormat, dict[tuple[int, int], ExpertEntry]]:
    """(format, index) of the routed experts under `model_path` (storage/index.py:182-193): a converted stacked affine
    bank when config.json says so, else the shipped FP4 layout."""
    root = Path(model_path)
    cfg = root / "config.json"
    if cfg.exists():
        try:
            spec = json.loads(cfg.read_text()).get("omlx_deepseek_v41")
        except (OSError, json.JSONDecodeError):
            spec = None
        if spec:
            return build_stacked_expert_index(root, spec.get("quantized_modules", {}))
    return FP4_FORMAT, build_expert_index(root)


def _dims(fmt: ExpertFormat, entry: ExpertEntry, headers: dict) -> tuple[int, int]:
    """(hidden, inter) of the bank."""
    if fmt.kind == "affine":
        inter, words = fmt.shapes["w1.weight"]
        return words * 32 // fmt.bits, inter
    for t in entry.tensors:
        if t.short == "w1.scale":
            inter, blocks = headers[t.shard][t.name]["shape"]
            return int(blocks) * 32, int(inter)
    raise ValueError("the index has no w1.scale tensor to take the bank's dimensions from")


def read_expert_into(entry: ExpertEntry, views: dict, fds: dict) -> int:
    """Reads one expert into writable buffers by short tensor name; tensors that follow one another in a shard go
    in one preadv.  Raises ValueError when a buffer's size is not the tensor's, OSError on a short read
    (storage/reader.py:182-260).  Returns the bytes read."""
    total = 0
    run: list[TensorRange] = []

    def flush():
        nonlocal total
        if not run:
            return
        bufs = []
        for t in run:
            target = memoryview(views[t.short]).cast("B")
            if target.nbytes != t.size:
                raise ValueError(f"slot buffer for {t.short} has {target.nbytes} bytes, tensor {t.name} has {t.size}")
            bufs.append(target)
        fd = fds.get(run[0].shard)
        if fd is None:
            fd = fds[run[0].shard] = os.open(run[0].shard, os.O_RDONLY)
        want = run[-1].end - run[0].start
        got = os.preadv(fd, bufs, run[0].start)
        if got != want:
            raise OSError(f"Short read from {run[0].shard}: expected {want}, got {got}")
        total += got
        run.clear()

    for t in entry.tensors:
        if run and (run[-1].shard != t.shard or run[-1].end != t.start):
            flush()
        run.append(t)
    flush()
    return total


def load_bank(model_path, device="cuda", *, layers=None, n_experts: int | None = None) -> SlabBank:
    """Every routed expert of the checkpoint (or of the given `layers`) as one resident `SlabBank`: slot
    layer_position * n_experts + expert, with the bank's slot table set accordingly.  An expert the checkpoint lacks
    keeps slot -1 (it contributes zeros).  Raises KeyError when nothing matches."""
    fmt, index = detect_expert_bank(model_path)
    if not index:
        raise KeyError(f"no routed experts found under {model_path}")
    all_layers = sorted({l for l, _ in index})
    layers = all_layers if layers is None else [l for l in layers if l in all_layers]
    if not layers:
        raise KeyError(f"none of the requested layers has routed experts under {model_path}")
    E = n_experts if n_experts is not None else max(e for _, e in index) + 1
    headers = {}
    if fmt.kind == "fp4":
        for shard, header, _ in _shards(Path(model_path)):
            headers[shard] = header
    hidden, inter = _dims(fmt, next(iter(index.values())), headers)
    bank = SlabBank(fmt, hidden, inter, len(layers) * E, layers=len(layers), n_experts=E, device=device)
    table = torch.full((len(layers), E), -1, dtype=torch.int32)
    on_gpu = bank.slab.is_cuda
    staging = [torch.empty(bank.record_bytes, dtype=torch.uint8, pin_memory=on_gpu) for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)] if on_gpu else None
    fds: dict = {}
    try:
        n = 0
        for li, layer in enumerate(layers):
            for e in range(E):
                entry = index.get((layer, e))
                if entry is None:
                    continue
                slot, buf = li * E + e, staging[n & 1]
                if on_gpu and n >= 2:
                    done[n & 1].synchronize()        # the copy that last used this staging record is over
                host = buf.numpy()
                views = {name: host[bank.offsets[name]:bank.offsets[name] + bank.tensor_sizes[name]] for name in fmt.tensor_names}
                missing = set(fmt.tensor_names) - {t.short for t in entry.tensors}
                if missing:
                    raise KeyError(f"expert {(layer, e)} lacks {sorted(missing)}")
                read_expert_into(entry, views, fds)
                bank.slab[slot].copy_(buf, non_blocking=on_gpu)
                if on_gpu:
                    done[n & 1].record()
                table[li, e] = slot
                n += 1
        if on_gpu:
            torch.cuda.synchronize(bank.slab.device)
    finally:
        for fd in fds.values():
            os.close(fd)
    bank.slot_table_host = table
    bank.slot_table = table.to(bank.slab.device)
    bank.calibrate_scale_centre()      # FP4: centre the grouped kernels' scale window on the bytes just loaded
    return bank
