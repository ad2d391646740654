"""Bringing a model's tensors from a store (a checkpoint, or seeded random values) to the device.

The model says which tensors it reads (``WeightDecl`` by full name); this
module checks the store against that list in one pass and raises ONE error
naming every missing tensor, every unexpected tensor and every wrong shape.
The reference fails on the first bad tensor (src/weight/weight_builder.cpp:
106-133) and ignores extras; listing them all at once is this engine's choice.

Storage types on the device:
  * integer tensors become int32;
  * with ``dtype=float32`` every floating tensor becomes float32;
  * with ``dtype=bfloat16`` matrices and tables become bfloat16, while a
    vector (rank <= 1) that the store holds in 32 bits stays in 32 bits
    (the norm kernels read their scale in either type).
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Mapping, Protocol

import torch

from ..config.errors import WeightError

# Roles choose the distribution of the random-weights mode.
ROLE_LINEAR = "linear"        # N(0, 0.02)
ROLE_NORM = "norm"            # 1 + N(0, 0.01)
ROLE_EMBEDDING = "embedding"  # N(0, 0.02)

_ROLE_INIT = {ROLE_LINEAR: (0.0, 0.02), ROLE_NORM: (1.0, 0.01), ROLE_EMBEDDING: (0.0, 0.02)}


@dataclass(frozen=True)
class WeightDecl:
    shape: tuple[int, ...]
    role: str = ROLE_LINEAR


class WeightStore(Protocol):
    def names(self) -> tuple[str, ...]: ...
    def shape(self, name: str) -> tuple[int, ...]: ...
    def dtype(self, name: str) -> torch.dtype: ...
    def read(self, name: str) -> torch.Tensor: ...


def check_store(store: WeightStore, expected: Mapping[str, WeightDecl], ignorable: tuple[str, ...] = ()) -> None:
    """Raise one ``WeightError`` listing missing and unexpected tensors and wrong shapes."""
    present = set(store.names())
    missing = sorted(name for name in expected if name not in present)
    unexpected = sorted(name for name in present if name not in expected and name not in ignorable)
    wrong = sorted((name, tuple(store.shape(name)), tuple(decl.shape)) for name, decl in expected.items()
                   if name in present and tuple(store.shape(name)) != tuple(decl.shape))
    not_float = sorted(name for name, decl in expected.items()
                       if name in present and not store.dtype(name).is_floating_point)
    if not (missing or unexpected or wrong or not_float):
        return
    lines = ["the checkpoint does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}):")
        lines += [f"    {name}  expected shape {list(expected[name].shape)}" for name in missing]
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}):")
        lines += [f"    {name}  shape {list(store.shape(name))}" for name in unexpected]
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}):")
        lines += [f"    {name}  found {list(found)}, expected {list(want)}" for name, found, want in wrong]
    if not_float:
        lines.append(f"  not floating point ({len(not_float)}):")
        lines += [f"    {name}  stored as {store.dtype(name)}" for name in not_float]
    raise WeightError("\n".join(lines))


def device_dtype(stored: torch.dtype, rank: int, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored == torch.float32 and rank <= 1:
        return torch.float32
    return engine_dtype


def load_weights(store: WeightStore, expected: Mapping[str, WeightDecl], dtype: torch.dtype,
                 device: torch.device | str, ignorable: tuple[str, ...] = ()) -> dict[str, torch.Tensor]:
    """Check the store, then bring every expected tensor to ``device`` in its storage type."""
    if dtype not in (torch.float32, torch.bfloat16):
        raise WeightError(f"engine dtype must be float32 or bfloat16, not {dtype}")
    check_store(store, expected, ignorable)
    out: dict[str, torch.Tensor] = {}
    for name, decl in expected.items():
        tensor = store.read(name)
        target = device_dtype(tensor.dtype, len(decl.shape), dtype)
        out[name] = tensor.to(device=device, dtype=target).contiguous()
    return out


# ------------------------------------------------------------------ random weights
def tensor_seed(seed: int, name: str) -> int:
    """A 63-bit seed for one tensor: the model seed mixed with a hash of the tensor's name."""
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & (2**63 - 1)


def random_tensor(seed: int, name: str, decl: WeightDecl, dtype: torch.dtype,
                  device: torch.device | str = "cpu") -> torch.Tensor:
    """Seeded values for one tensor.  Each tensor has its own key, so the value of a tensor does not
    depend on which other tensors exist or in which order they are made.  On a CUDA device this
    package's counter-based fill kernel writes them straight in ``dtype`` (no float32 copy of the
    tensor; the reference fills random models with a kernel of its own too,
    deps/ttl/src/kernels/random/random.cu:83-125); on the CPU torch's generator draws them in float32
    and they are rounded.  The two give different streams: a model folder holds whatever made it."""
    if decl.role not in _ROLE_INIT:
        raise WeightError(f"tensor '{name}' has the unknown role {decl.role!r}")
    mean, std = _ROLE_INIT[decl.role]
    if torch.device(device).type == "cuda" and dtype in (torch.bfloat16, torch.float32):
        from ..kernels import ops
        with torch.cuda.device(device):
            return ops.fill_normal(torch.empty(decl.shape, dtype=dtype, device=device), tensor_seed(seed, name), mean, std)
    generator = torch.Generator(device=device)
    generator.manual_seed(tensor_seed(seed, name))
    values = torch.randn(decl.shape, generator=generator, dtype=torch.float32, device=device)
    return values.mul_(std).add_(mean).to(dtype)


class RandomWeights:
    """A weight store of seeded random tensors, made where they are read (no file, no host copy)."""

    def __init__(self, expected: Mapping[str, WeightDecl], seed: int, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device | str = "cpu"):
        self._expected = dict(expected)
        self._seed = seed
        self._dtype = dtype
        self._device = device

    def names(self) -> tuple[str, ...]:
        return tuple(self._expected)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._expected[name].shape)

    def dtype(self, name: str) -> torch.dtype:
        return self._dtype

    def read(self, name: str) -> torch.Tensor:
        return random_tensor(self._seed, name, self._expected[name], self._dtype, self._device)
