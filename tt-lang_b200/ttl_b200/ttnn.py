"""`ttnn` surface of the B200 backend.

Mirrors the subset of TT-NN that tt-lang programs use, with the names and argument
meanings of the reference simulator's stand-in (python/sim/ttnnsim.py:113-226,
521-580, 583-771).  A Tensor wraps a row-major torch tensor that lives in the HBM
of the current CUDA device; "tiles" are an indexing convention (tile (r, c) is the
element window [32r:32r+32, 32c:32c+32], python/sim/tensoraccessor.py:125-159).
On a machine without a GPU tensors stay on the host so that programs can still be
traced and recognised; launching them raises.
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple, Union

import torch

from .symloop import NeedsConcrete as _NeedsConcrete
from .symloop import SymInt as _SymInt
from .symloop import const_extent as _const_extent
from .symloop import live_sites as _live_sites

TILE_SIZE: int = 32
TILE_SHAPE: Tuple[int, int] = (32, 32)
TILE_LAYOUT = "TILE"
ROW_MAJOR_LAYOUT = "ROW_MAJOR"
L1_MEMORY_CONFIG = None
DRAM_MEMORY_CONFIG = None

bfloat16 = torch.bfloat16
float32 = torch.float32


class _BlockFloat8:
    """Marker dtype for bfloat8_b (1088-byte tiles; python/ttl/dtype_utils.py:174-175)."""

    def __repr__(self) -> str:
        return "ttnn.bfloat8_b"


bfloat8_b = _BlockFloat8()


class _BlockFloat4:
    """Marker dtype for bfloat4_b (576-byte tiles; python/ttl/dtype_utils.py:178-179)."""

    def __repr__(self) -> str:
        return "ttnn.bfloat4_b"


bfloat4_b = _BlockFloat4()

Shape = Tuple[int, ...]


def _default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


class CoreCoord:
    """Core coordinate (python/sim/ttnnsim.py:120-139)."""

    def __init__(self, x: int, y: int):
        self.x = x
        self.y = y

    def __repr__(self) -> str:
        return f"CoreCoord(x={self.x}, y={self.y})"

    def __eq__(self, other: object) -> bool:
        return isinstance(other, CoreCoord) and self.x == other.x and self.y == other.y

    def __hash__(self) -> int:
        return hash((self.x, self.y))


class CoreRange:
    """Inclusive rectangle of cores (python/sim/ttnnsim.py:142-161)."""

    def __init__(self, start: CoreCoord, end: CoreCoord):
        self.start = start
        self.end = end

    def __repr__(self) -> str:
        return f"CoreRange(start={self.start}, end={self.end})"

    def num_cores(self) -> int:
        return (self.end.x - self.start.x + 1) * (self.end.y - self.start.y + 1)


class CoreRangeSet:
    """Collection of core ranges (python/sim/ttnnsim.py:164-186)."""

    def __init__(self, ranges: List[CoreRange]):
        self._ranges = list(ranges)

    def ranges(self) -> List[CoreRange]:
        return self._ranges

    def num_cores(self) -> int:
        return sum(r.num_cores() for r in self._ranges)

    def __repr__(self) -> str:
        return f"CoreRangeSet(ranges={self._ranges})"


class Device:
    """Handle for one GPU.  `compute_with_storage_grid_size` keeps the simulator's
    8x8 answer (python/sim/ttnnsim.py:206-215): the grid only decides how a tile
    program splits its own loops, not how the GPU kernel is scheduled."""

    def __init__(self, device_id: int = 0) -> None:
        self.device_id = device_id

    def __repr__(self) -> str:
        return f"Device(id={self.device_id})"

    def compute_with_storage_grid_size(self) -> CoreCoord:
        return CoreCoord(8, 8)


def open_device(device_id: int = 0) -> Device:
    if torch.cuda.is_available():
        torch.cuda.set_device(device_id)
    return Device(device_id)


def close_device(device: Device) -> None:
    return None


def _tile_dim(n: int) -> int:
    return 1 if n == 1 else n // TILE_SIZE


def _extent(sl: slice, what: str) -> int:
    return _const_extent(sl.start, sl.stop, what)


def _bounds(x: Any) -> Tuple[int, int]:
    """(smallest, largest) value of a tile index."""
    if isinstance(x, _SymInt):
        return int(x.v.min()), int(x.v.max())
    return int(x), int(x)


class Tensor:
    """Row-major 2-D tensor in device memory.

    `t[r0:r1, c0:c1]` with tile coordinates returns a view that remembers where it
    came from, which is what `ttl.copy` needs; everything else behaves like the
    simulator's Tensor (python/sim/ttnnsim.py:229-519).
    """

    def __init__(self, tensor: torch.Tensor, *, _origin: Optional[Tuple["Tensor", int, int, int, int]] = None,
                 _packed: Optional[torch.Tensor] = None, _logical_shape: Optional[Shape] = None,
                 _packed_bits: int = 8) -> None:
        self._t = tensor                # None for a tile view whose torch view has not been asked for yet
        self._origin = _origin          # (base tensor, r0, r1, c0, c1) in tiles
        self._packed = _packed          # block-float payload (uint8: 1088 bytes per bfloat8_b tile, 576 per bfloat4_b tile)
        self._packed_bits = _packed_bits
        self._logical_shape = _logical_shape

    # -- basic properties ------------------------------------------------
    @property
    def _tensor(self) -> torch.Tensor:
        """The torch tensor; for a tile view made by indexing, the torch view is created on first use (a tile
        program indexes a tensor once per copy and only ever hands the view to ttl.copy)."""
        t = self._t
        if t is None:
            base, r0, r1, c0, c1 = self._origin  # type: ignore[misc]
            t = self._t = base._tensor[int(r0) * TILE_SIZE:int(r1) * TILE_SIZE, int(c0) * TILE_SIZE:int(c1) * TILE_SIZE]
        return t

    @_tensor.setter
    def _tensor(self, value: torch.Tensor) -> None:
        self._t = value

    @property
    def shape(self) -> Shape:
        if self._logical_shape is not None:
            return tuple(self._logical_shape)
        return tuple(self._tensor.shape)

    @property
    def dtype(self) -> Any:
        if self._packed is not None:
            return bfloat8_b if self._packed_bits == 8 else bfloat4_b
        if self._t is None:
            return self._origin[0].dtype  # type: ignore[index]
        return self._t.dtype

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype})"

    def memory_config(self) -> Any:
        """Everything lives in HBM; the L1 / DRAM distinction of the reference has no counterpart."""
        return DRAM_MEMORY_CONFIG

    def to_torch(self) -> torch.Tensor:
        return to_torch(self)

    def tile_shape(self) -> Tuple[int, int]:
        """Shape in tiles; a size-1 dim counts as one (degenerate) tile
        (python/sim/tensoraccessor.py:209-216)."""
        return (_tile_dim(self.shape[0]), _tile_dim(self.shape[1]))

    def _is_tile_indexable(self) -> bool:
        if len(self.shape) != 2:
            return False
        return all(d == 1 or d % TILE_SIZE == 0 for d in self.shape)

    # -- tile indexing ---------------------------------------------------
    @staticmethod
    def _norm(index: Any, name: str) -> slice:
        if isinstance(index, (int, _SymInt)):
            return slice(index, index + 1)
        if index.start is None:
            raise ValueError(
                f"Slice {name} must have explicit start value, got slice({index.start}, {index.stop}, {index.step})")
        if index.stop is None:
            raise ValueError(
                f"Slice {name} must have explicit stop value, got slice({index.start}, {index.stop}, {index.step})")
        if index.step is not None:
            raise ValueError(
                f"Slice {name} must not have step value, got slice({index.start}, {index.stop}, {index.step}). "
                "Only simple slices are supported.")
        return index

    def _tile_view(self, key: Tuple[Any, Any]) -> "Tensor":
        if len(self.shape) != 2:
            raise ValueError("Tile-style indexing requires a 2D tensor")   # python/sim/ttnnsim.py:364-366
        if not self._is_tile_indexable():
            for i, d in enumerate(self.shape):
                if d != 1 and d % TILE_SIZE != 0:
                    raise ValueError(
                        f"Tensor dimension {i} has size {d} which is not a multiple of tile dimension {TILE_SIZE}")
            raise ValueError("Tile-style indexing requires a 2D tensor")
        rs = self._norm(key[0], "row")
        cs = self._norm(key[1], "col")
        base, br, _, bc, _ = self._origin if self._origin is not None else (self, 0, 0, 0, 0)
        origin = (base, br + rs.start, br + rs.stop, bc + cs.start, bc + cs.stop)
        symbolic = any(isinstance(x, _SymInt) for x in (rs.start, rs.stop, cs.start, cs.stop))
        if self._packed is not None:
            return Tensor(self._t, _origin=origin, _packed=self._packed, _packed_bits=self._packed_bits,
                          _logical_shape=(_extent(rs, "a tile view") * TILE_SIZE, _extent(cs, "a tile view") * TILE_SIZE))
        if self._origin is None:
            # a window of a whole tensor: only its shape is worked out now (what slicing would give)
            shape = []
            for sl, n in ((rs, self.shape[0]), (cs, self.shape[1])):
                if symbolic:
                    lo, hi = _bounds(sl.start), _bounds(sl.stop)
                    if lo[0] < 0 or hi[1] * TILE_SIZE > max(n, TILE_SIZE):
                        raise _NeedsConcrete(_live_sites(), "a tile index leaves the tensor")
                    shape.append(1 if n == 1 else _extent(sl, "a tile view") * TILE_SIZE)
                elif sl.start < 0 or sl.stop < 0:
                    shape = []
                    break
                else:
                    shape.append(max(0, min(n, sl.stop * TILE_SIZE) - min(n, sl.start * TILE_SIZE)))
            if shape:
                return Tensor(None, _origin=origin, _logical_shape=tuple(shape))  # type: ignore[arg-type]
        if symbolic:
            raise _NeedsConcrete(_live_sites(), "a view of a tile view is indexed with the loop variable")
        view = self._tensor[rs.start * TILE_SIZE:rs.stop * TILE_SIZE, cs.start * TILE_SIZE:cs.stop * TILE_SIZE]
        return Tensor(view, _origin=origin)

    def __getitem__(self, key: Any) -> "Tensor":
        if isinstance(key, tuple) and len(key) == 2:
            rk, ck = key
            if isinstance(rk, int) and isinstance(ck, int) and not self._is_tile_indexable():
                return Tensor(self._tensor[key])
            if isinstance(rk, (slice, int, _SymInt)) and isinstance(ck, (slice, int, _SymInt)):
                return self._tile_view(key)
        return Tensor(self._tensor[key])

    def __setitem__(self, key: Any, value: Any) -> None:
        v = value._tensor if isinstance(value, Tensor) else value
        if isinstance(key, tuple) and len(key) == 2:
            rk, ck = key
            if isinstance(rk, (slice, int)) and isinstance(ck, (slice, int)) and self._is_tile_indexable():
                self._tile_view(key)._tensor[...] = v
                return
        self._tensor[key] = v

    # -- eager element-wise arithmetic (used by programs for their golden results)
    def _bin(self, other: Any, fn: Any) -> "Tensor":
        if isinstance(other, Tensor):
            return Tensor(fn(self._tensor, other._tensor))
        if isinstance(other, (int, float)):
            return Tensor(fn(self._tensor, other))
        return NotImplemented

    def __add__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a + b)
    def __sub__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a - b)
    def __mul__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a * b)
    def __truediv__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a / b)
    def __floordiv__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a // b)
    def __mod__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a % b)
    def __pow__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: a ** b)
    def __radd__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: b + a)
    def __rsub__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: b - a)
    def __rmul__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: b * a)
    def __rtruediv__(self, o: Any) -> "Tensor": return self._bin(o, lambda a, b: b / a)

    def __matmul__(self, o: Any) -> "Tensor":
        if isinstance(o, Tensor):
            return Tensor(self._tensor @ o._tensor)
        return NotImplemented


def rand(shape: Shape, dtype: torch.dtype = bfloat16, layout: Any = TILE_LAYOUT) -> Tensor:
    """Uniform [0,1) tensor, generated in fp32 on the host and cast, exactly as the
    simulator does (python/sim/ttnnsim.py:521-531) so that seeds give the same values."""
    t = torch.rand(shape, dtype=torch.float32).to(dtype)
    return Tensor(t.to(_default_device()))


def empty(shape: Shape, dtype: torch.dtype = bfloat16, layout: Any = TILE_LAYOUT) -> Tensor:
    return Tensor(torch.empty(shape, dtype=dtype, device=_default_device()))


def zeros(shape: Shape, dtype: torch.dtype = bfloat16, layout: Any = TILE_LAYOUT) -> Tensor:
    return Tensor(torch.zeros(shape, dtype=dtype, device=_default_device()))


def to_torch(t: Union[Tensor, torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Host copy of a tensor (a device-to-host transfer when the tensor is in HBM).
    `out` (an extension over the reference signature) names a host tensor to fill, e.g. a
    pinned buffer, instead of allocating a pageable one; the call returns after the copy."""
    if isinstance(t, Tensor):
        if t._packed is not None:
            from .bfp8 import unpack_bfp4_b, unpack_bfp8_b
            return (unpack_bfp8_b if t._packed_bits == 8 else unpack_bfp4_b)(t._packed.cpu(), t.shape[0], t.shape[1])
        if out is not None:
            out.copy_(t._tensor, non_blocking=True)
            if t._tensor.is_cuda:
                torch.cuda.current_stream(t._tensor.device).synchronize()
                _check_device_status(t._tensor.device)
            return out
        host = t._tensor.cpu()
        if t._tensor.is_cuda:
            _check_device_status(t._tensor.device)
        return host
    if isinstance(t, torch.Tensor):
        return t.cpu()
    raise TypeError(f"Unsupported type for to_torch: {type(t)}")


def _check_device_status(device: torch.device) -> None:
    """Reading results back is where the host already waits for the GPU: raise here if a bounded device-side wait
    of a kernel launched on that GPU ran out (the kernel unwound and left its output partly written)."""
    from . import capi

    ctx = capi._CONTEXTS.get(device.index)
    if ctx is not None:
        ctx.check_status(int(torch.cuda.current_stream(device).cuda_stream))


def from_torch(tensor: torch.Tensor, dtype: Any = None, layout: Any = None, device: Optional[Device] = None,
               memory_config: Any = None) -> Tensor:
    """Move a host tensor into device memory (host-to-device transfer), converting the
    element type first when `dtype` is given (python/sim/ttnnsim.py:554-580).
    dtype=ttnn.bfloat8_b packs the tensor into 1088-byte block-float tiles."""
    dev = _default_device()
    if device is not None and torch.cuda.is_available():
        dev = torch.device("cuda", device.device_id)
    if isinstance(dtype, (_BlockFloat8, _BlockFloat4)):
        from .bfp8 import pack_bfp4_b, pack_bfp8_b
        if tensor.dim() != 2 or tensor.shape[0] % TILE_SIZE or tensor.shape[1] % TILE_SIZE:
            raise ValueError(f"{dtype!r} needs a 2-D tensor whose dims are multiples of 32")
        bits = 8 if isinstance(dtype, _BlockFloat8) else 4
        packed = (pack_bfp8_b if bits == 8 else pack_bfp4_b)(tensor.detach().to(torch.float32).cpu().contiguous())
        return Tensor(torch.empty(0), _packed=packed.to(dev, non_blocking=True),
                      _logical_shape=tuple(tensor.shape), _packed_bits=bits)
    if dtype is not None and tensor.dtype != dtype:
        tensor = tensor.to(dtype)
    return Tensor(tensor.to(dev, non_blocking=True))


def to_memory_config(t: Tensor, memory_config: Any = None, **_: Any) -> Tensor:
    """Identity: there is one memory space (HBM)."""
    return t


def squeeze(input_tensor: Tensor, dim: Optional[int] = None) -> Tensor:
    x = input_tensor._tensor
    return Tensor(x.squeeze() if dim is None else x.squeeze(dim))


def repeat(input_tensor: Tensor, repeats: Any) -> Tensor:
    return Tensor(input_tensor._tensor.repeat(*tuple(repeats)))


def multiply(a: Tensor, b: Tensor) -> Tensor:
    return a * b


def add(a: Tensor, b: Tensor) -> Tensor:
    return a + b


def isclose(a: Tensor, b: Tensor, rtol: float = 1e-5, atol: float = 1e-8) -> Tensor:
    return Tensor(torch.isclose(a._tensor, b._tensor, rtol=rtol, atol=atol))


def split_work_to_cores(core_grid: Union[CoreCoord, CoreRangeSet], units_to_divide: int, row_wise: bool = False):
    """Divide `units_to_divide` work units over a core grid: the first `remainder`
    cores (group 1) get one unit more than the rest (group 2).  Same contract and
    core ordering as python/sim/ttnnsim.py:583-752."""
    if isinstance(core_grid, CoreCoord):
        gx, gy = core_grid.x, core_grid.y
        if row_wise:
            order = [CoreCoord(x, y) for y in range(gy) for x in range(gx)]
        else:
            order = [CoreCoord(x, y) for x in range(gx) for y in range(gy)]
        all_cores = CoreRangeSet([CoreRange(CoreCoord(0, 0), CoreCoord(gx - 1, gy - 1))])
    else:
        order = [CoreCoord(x, y) for r in core_grid.ranges()
                 for y in range(r.start.y, r.end.y + 1) for x in range(r.start.x, r.end.x + 1)]
        all_cores = core_grid
    used = min(len(order), units_to_divide)
    if used == 0:
        e = CoreRangeSet([])
        return 0, e, e, e, 0, 0
    base, rem = divmod(units_to_divide, used)
    if rem:
        n1, u1, u2 = rem, base + 1, base
    else:
        n1, u1, u2 = used, base, 0
    g1 = CoreRangeSet([CoreRange(c, c) for c in order[:n1]])
    g2 = CoreRangeSet([CoreRange(c, c) for c in order[n1:used]])
    return used, all_cores, g1, g2, u1, u2
