"""Expert bank in HBM: slot records, the (layer, expert) -> slot table and per-expert accessors.

Device-side counterpart of the reference's slot store for a machine where every expert is
resident: `SlabBank` is the slab pool (cache/slots.py:185-251: records of fixed size with
fixed per-tensor offsets), `ExpertFormat` / `FP4_FORMAT` follow storage/index.py:41-67,
`ResidentExpert` follows cache/resident.py:11-52, and `slot_table` is the int32
[layers, experts] table of cache/resident_store.py:637-646 (-1 = not resident).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib

TENSOR_NAMES_FP4 = ("w1.weight", "w1.scale", "w2.weight", "w2.scale", "w3.weight", "w3.scale")
TENSOR_NAMES_AFFINE = (
    "w1.weight", "w1.scales", "w1.biases",
    "w2.weight", "w2.scales", "w2.biases",
    "w3.weight", "w3.scales", "w3.biases",
)
_ALIGN = 256


@dataclass(frozen=True)
class ExpertFormat:
    """How a routed expert's slot bytes are laid out and multiplied (storage/index.py:41-57)."""

    kind: str                      # "fp4" or "affine"
    bits: int
    group_size: int
    tensor_names: tuple[str, ...]
    shapes: dict = field(default_factory=dict)
    dtypes: dict = field(default_factory=dict)


FP4_FORMAT = ExpertFormat(kind="fp4", bits=4, group_size=32, tensor_names=TENSOR_NAMES_FP4)


def affine_format(hidden: int, inter: int, bits: int = 2, group_size: int = 128, scale_dtype: str = "float16") -> ExpertFormat:
    """Format of a stacked affine bank.  Scales/biases have one entry per `group_size` consecutive
    elements of the flattened [N*K] weight, which is the reference's [N, K/group] whenever the
    group divides K (it does for the reference's 5120/2304; 2880 is 22.5 groups of 128)."""
    shapes, dtypes = {}, {}
    for proj, (n, k) in (("w1", (inter, hidden)), ("w2", (hidden, inter)), ("w3", (inter, hidden))):
        shapes[f"{proj}.weight"] = (n, k * bits // 32)
        dtypes[f"{proj}.weight"] = "uint32"
        groups = (n, k // group_size) if k % group_size == 0 else (n * k // group_size,)
        for f in ("scales", "biases"):
            shapes[f"{proj}.{f}"] = groups
            dtypes[f"{proj}.{f}"] = scale_dtype
    return ExpertFormat("affine", bits, group_size, TENSOR_NAMES_AFFINE, shapes, dtypes)


def tensor_sizes(fmt: ExpertFormat, hidden: int, inter: int) -> dict[str, int]:
    """Bytes of each tensor of one expert record."""
    dims = {"w1": (inter, hidden), "w2": (hidden, inter), "w3": (inter, hidden)}
    out = {}
    for name in fmt.tensor_names:
        n, k = dims[name[:2]]
        if fmt.kind == "fp4":
            out[name] = n * k // 2 if name.endswith("weight") else n * k // 32
        else:
            out[name] = n * k * fmt.bits // 8 if name.endswith("weight") else (n * k // fmt.group_size) * 2
    return out


_TORCH_DT = {"uint8": torch.uint8, "uint32": torch.int32, "float16": torch.float16, "bfloat16": torch.bfloat16}


class SlabBank:
    """`n_slots` expert records in one uint8 [n_slots, record_bytes] device tensor."""

    def __init__(self, fmt: ExpertFormat, hidden: int, inter: int, n_slots: int, *, layers: int = 1,
                 n_experts: int | None = None, device="cuda", storage: torch.Tensor | None = None) -> None:
        if n_slots <= 0:
            raise ValueError(f"n_slots must be positive, got {n_slots}")
        self.fmt, self.hidden, self.inter, self.n_slots = fmt, int(hidden), int(inter), int(n_slots)
        self.tensor_sizes = tensor_sizes(fmt, hidden, inter)
        self.offsets: dict[str, int] = {}
        pos = 0
        for name in fmt.tensor_names:
            self.offsets[name] = pos
            pos += -(-self.tensor_sizes[name] // _ALIGN) * _ALIGN
        self.record_bytes = pos
        if storage is None:
            storage = torch.zeros((n_slots, self.record_bytes), dtype=torch.uint8, device=device)
        if storage.dtype != torch.uint8 or tuple(storage.shape) != (n_slots, self.record_bytes):
            raise ValueError(f"storage must be uint8 [{n_slots}, {self.record_bytes}], got {storage.dtype} {tuple(storage.shape)}")
        self.slab = storage
        self.layers = int(layers)
        self.n_experts = int(n_experts) if n_experts is not None else n_slots // max(1, self.layers)
        # identity table for an all-resident bank: (layer, expert) -> layer * E + expert
        table = torch.full((self.layers, self.n_experts), -1, dtype=torch.int32)
        flat = torch.arange(min(self.layers * self.n_experts, n_slots), dtype=torch.int32)
        table.view(-1)[: flat.numel()] = flat
        self.slot_table_host = table                      # host copy for Python-side lookups
        self.slot_table = table.to(self.slab.device)      # device copy for the routing kernel
        d = _lib.BankDesc()
        d.record_bytes = self.record_bytes
        for i, name in enumerate(fmt.tensor_names):
            d.off[i] = self.offsets[name]
        d.n_slots, d.hidden, d.inter = self.n_slots, self.hidden, self.inter
        d.format = _lib.BANK_FP4 if fmt.kind == "fp4" else _lib.BANK_AFFINE
        d.bits, d.group = fmt.bits, fmt.group_size
        sdt = fmt.dtypes.get("w1.scales", "float16")
        d.scale_dtype = _lib.BF16 if sdt == "bfloat16" else _lib.F16
        d.fp4_scale_centre = 0
        self.desc = d
        self._scale_lo, self._scale_hi = 255, 0      # E8M0 bytes seen so far (FP4 banks; byte 0 is not counted)

    def _note_scale_bytes(self, lo: int, hi: int) -> None:
        """Widens the range of E8M0 bytes the bank is known to hold and re-centres the descriptor on it."""
        self._scale_lo, self._scale_hi = min(self._scale_lo, lo), max(self._scale_hi, hi)
        if self._scale_hi - self._scale_lo > 27:
            raise NotImplementedError(f"FP4 block scales span 2**{self._scale_lo - 127}..2**{self._scale_hi - 127}: "
                                      "wider than the 28 binades the grouped kernels hold in f16")
        self.desc.fp4_scale_centre = max(1, min(254, (self._scale_lo + self._scale_hi + 1) // 2))

    def calibrate_scale_centre(self) -> int:
        """FP4 banks: set the descriptor's scale centre to the middle of the E8M0 bytes actually
        stored (the tensor-core kernels hold block scales relative to it in f16 and accept
        centre-14 .. centre+13).  Call once after the bank is filled; returns the centre."""
        if self.fmt.kind != "fp4":
            return 0
        self._scale_lo, self._scale_hi = 255, 0
        for name in ("w1.scale", "w2.scale", "w3.scale"):
            o, n = self.offsets[name], self.tensor_sizes[name]
            region = self.slab[:, o:o + n]
            # byte 0 (2**-127) marks a block that is zero whatever its codes are; it does not widen the range
            nz = torch.where(region == 0, torch.full_like(region, 255), region)
            self._note_scale_bytes(int(nz.min()), int(region.max()))
        return int(self.desc.fp4_scale_centre)

    @property
    def desc_ptr(self):
        return C.byref(self.desc)

    @property
    def nbytes(self) -> int:
        return self.n_slots * self.record_bytes

    @property
    def expert_bytes(self) -> int:
        """Algorithmic bytes of one expert (padding excluded)."""
        return sum(self.tensor_sizes.values())

    def view(self, slot: int, name: str) -> torch.Tensor:
        """Zero-copy uint8 view of one tensor of one slot; stays valid across refills of the slot."""
        o = self.offsets[name]
        return self.slab[slot, o:o + self.tensor_sizes[name]]

    def typed_view(self, slot: int, name: str) -> torch.Tensor:
        v = self.view(slot, name)
        if self.fmt.kind == "affine":
            return v.view(_TORCH_DT[self.fmt.dtypes[name]]).reshape(self.fmt.shapes[name])
        n, k = {"w1": (self.inter, self.hidden), "w2": (self.hidden, self.inter), "w3": (self.inter, self.hidden)}[name[:2]]
        return v.reshape(n, k // 2 if name.endswith("weight") else k // 32)

    def write_expert(self, slot: int, tensors: dict) -> None:
        """Copy one expert's tensors (numpy arrays or torch tensors, any device) into a slot."""
        import numpy as np

        if not 0 <= slot < self.n_slots:
            raise KeyError(f"slot {slot} outside [0, {self.n_slots})")
        for name in self.fmt.tensor_names:
            src = tensors[name]
            if isinstance(src, np.ndarray):
                src = torch.from_numpy(np.ascontiguousarray(src).view(np.uint8).reshape(-1))
            else:
                src = src.contiguous().view(torch.uint8).reshape(-1)
            if src.numel() != self.tensor_sizes[name]:
                raise ValueError(f"{name}: {src.numel()} bytes, slot expects {self.tensor_sizes[name]}")
            if self.fmt.kind == "fp4" and name.endswith(".scale") and src.numel():
                # keep the descriptor's scale centre on the bytes the bank holds (the grouped FP4 kernels clamp
                # scales outside centre-14 .. centre+13); byte 0 = a zero block, not counted
                nz = torch.where(src == 0, torch.full_like(src, 255), src)
                lo, hi = int(nz.min()), int(src.max())
                if lo <= hi:
                    self._note_scale_bytes(lo, hi)
            self.view(slot, name).copy_(src)

    def fill_random(self, gen: torch.Generator | None = None, step: int = 64) -> None:
        """Fills every slot with synthetic weights of the benchmark's distributions: uniform codes; FP4
        block scales uniform in 2**-9 .. 2**-4; affine scales ~U(0.002, 0.02) and biases ~N(0, 0.01)."""
        dev = self.slab.device
        for s0 in range(0, self.n_slots, step):
            s1 = min(s0 + step, self.n_slots)
            for name in self.fmt.tensor_names:
                o, n = self.offsets[name], self.tensor_sizes[name]
                region = self.slab[s0:s1, o:o + n]
                if name.endswith("weight"):
                    region.copy_(torch.randint(0, 256, (s1 - s0, n), dtype=torch.uint8, device=dev, generator=gen))
                elif self.fmt.kind == "fp4":
                    region.copy_(torch.randint(118, 124, (s1 - s0, n), dtype=torch.uint8, device=dev, generator=gen))
                elif name.endswith("scales"):
                    v = torch.rand((s1 - s0, n // 2), device=dev, generator=gen) * 0.018 + 0.002
                    region.view(torch.float16).copy_(v.to(torch.float16))
                else:
                    v = torch.randn((s1 - s0, n // 2), device=dev, generator=gen) * 0.01
                    region.view(torch.float16).copy_(v.to(torch.float16))
        if self.fmt.kind == "fp4":
            self._note_scale_bytes(118, 123)

    def expert(self, layer: int, expert: int) -> "ResidentExpert":
        in_range = 0 <= layer < self.layers and 0 <= expert < self.n_experts
        slot = int(self.slot_table_host[layer, expert]) if in_range else -1
        if slot < 0:
            raise KeyError(f"Missing expert entry: {(layer, expert)!r}")
        return ResidentExpert(layer, expert, slot, self)


@dataclass(eq=False)
class ResidentExpert:
    """A routed expert living in a bank slot; the arrays alias the slot's memory."""

    layer: int
    expert: int
    slot: int
    bank: SlabBank

    def _t(self, name: str) -> torch.Tensor:
        return self.bank.view(self.slot, name)

    w1_weight = property(lambda s: s._t("w1.weight"))
    w1_scale = property(lambda s: s._t("w1.scale"))
    w2_weight = property(lambda s: s._t("w2.weight"))
    w2_scale = property(lambda s: s._t("w2.scale"))
    w3_weight = property(lambda s: s._t("w3.weight"))
    w3_scale = property(lambda s: s._t("w3.scale"))

    @property
    def size(self) -> int:
        return self.bank.expert_bytes

    @property
    def key(self) -> tuple[int, int]:
        return (self.layer, self.expert)

    def as_model_dict(self) -> dict[str, torch.Tensor]:
        return {n: self._t(n) for n in self.bank.fmt.tensor_names}
