"""Executor API of gint, backed by the B200 kernels (mirror of ``gint/host/executor.py`` +
``gint/host/cuda/executor_impl.py``).

Public names, argument meaning and error behaviour follow the reference so that programs, tests and the
conductor's ``executor.execute(program, tensor_interfaces, grid_dim, cuda_stream=...)`` calls work unchanged:

* ``ProgramTensorInfo`` / ``ProgramData`` / ``TensorInterface``  (``executor.py:14-98``)
* ``BaseExecutableProgram`` with ``get_program`` / ``cache_policy`` / ``__call__(*, grid_dim)``  (``executor.py:152-197``)
* ``BaseExecutor.{warp_size, execute, execute_indirect}`` and the ``get_executor()`` singleton  (``executor.py:200-233``)

What differs is below the seam: ``B200Executor`` hands the bytecode and the descriptor template to
``libgint_b200.so`` once per (program, cache key, device) and each later call is one C call that patches base
pointers into kernel parameters and launches. There is no CPU path.
"""
from __future__ import annotations

import ctypes
import sys
import threading
from collections.abc import Hashable
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence, Union

import numpy
import torch

from ..opcodes import MAX_N_TENSORS, REG_WIDTH
from . import capi
from .analyzer import BytecodeStats, analyze_bytecode, select_pool_size
from .utils import fill_tensor_info

# Kernel geometries of the reference, kept for callers that ask by name (``gint/kernel/interpreter/main.py:34-38``):
# name -> (pool size, registers, max stack).
VARIANTS: dict[str, tuple[int, int, int]] = {"s7": (7, 4, 7), "l12": (12, 8, 8)}
DEFAULT_VARIANT = "l12"


@dataclass
class ProgramTensorInfo:
    elm_size: int
    batch_strides: list[int]
    batch_shape: list[int]
    block_shape_stride_1: list[int]
    block_shape_stride_2: list[int]
    block_grid_dims: list[int]
    block_grid_steps: list[int]


@dataclass
class ProgramData:
    program: numpy.ndarray            # int32, flat [opcode, operand, opcode, operand, ...]
    input_infos: list[ProgramTensorInfo]
    input_indices: Optional[list[int]] = None   # descriptor slot i reads argument input_indices[i]
    _stats: Optional[BytecodeStats] = field(default=None, repr=False, compare=False)

    @property
    def stats(self) -> BytecodeStats:
        if self._stats is None:
            self._stats = analyze_bytecode(self.program)
        return self._stats


@dataclass
class TensorInterface:
    typechr: str
    elm_size: int
    base_ptr: int
    shape: tuple[int, ...]
    strides: tuple[int, ...]   # in elements

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def typestr(self) -> str:
        return f"{self.typechr}{self.elm_size}"

    @property
    def __cuda_array_interface__(self) -> dict:
        return {"version": 2, "data": (self.base_ptr, False), "shape": self.shape,
                "typestr": f"<{self.typechr}{self.elm_size}", "strides": tuple(s * self.elm_size for s in self.strides)}

    @classmethod
    def from_cuda_array_interface(cls, obj: Union[dict, Any]) -> "TensorInterface":
        cai = obj if isinstance(obj, dict) else getattr(obj, "__cuda_array_interface__", None)
        if cai is None:
            raise TypeError("__cuda_array_interface__ not found for cuda array interface object.")
        if "typestr" not in cai:
            raise TypeError("Invalid __cuda_array_interface__: missing `typestr`")
        typestr = cai["typestr"]
        if typestr[0] not in "<|" or sys.byteorder != "little":
            raise AssertionError("gint does not support big endian yet")
        if cai["version"] < 2:
            raise AssertionError(cai["version"])
        ptr, readonly = cai["data"]
        if readonly:
            raise AssertionError("gint does not support readonly")
        nbytes = int(typestr[2:])
        shape = tuple(cai["shape"])
        if cai.get("strides"):
            strides = tuple(s // nbytes for s in cai["strides"])
        else:
            strides, acc = [], 1
            for extent in reversed(shape):
                strides.append(acc)
                acc *= extent
            strides = tuple(reversed(strides))
        if len(shape) != len(strides):
            raise AssertionError((shape, strides, "shape and strides must have the same ndim"))
        return cls(typestr[1], nbytes, ptr, shape, strides)


_TORCH_TYPES = {
    torch.float32: ("f", 4), torch.float16: ("f", 2), torch.bfloat16: ("f", 2), torch.float64: ("f", 8),
    torch.int32: ("i", 4), torch.int64: ("i", 8), torch.uint8: ("u", 1), torch.bool: ("b", 1),
}


def _convert_arg(arg) -> TensorInterface:
    if isinstance(arg, TensorInterface):
        return arg
    if isinstance(arg, torch.Tensor):
        typechr, size = _TORCH_TYPES[arg.dtype]
        return TensorInterface(typechr, size, arg.data_ptr(), tuple(arg.shape), tuple(arg.stride()))
    return TensorInterface.from_cuda_array_interface(arg)


def select_variant(bytecode_or_pd) -> str:
    """Name of the reference kernel geometry that would run this program (``gint/host/executor.py:131-149``).
    The B200 library chooses its own pool size (``ProgramData.stats`` -> ``select_pool_size``); this is for callers
    and tests that reason in the reference's terms."""
    stats = bytecode_or_pd.stats if isinstance(bytecode_or_pd, ProgramData) else analyze_bytecode(bytecode_or_pd)
    for name, (_, regs, stack) in sorted(VARIANTS.items(), key=lambda kv: kv[1][0]):
        if stats.max_stack <= stack and stats.max_reg_idx + 1 <= regs:
            return name
    return DEFAULT_VARIANT


class BaseExecutableProgram:
    REGW = REG_WIDTH

    def get_program(self, *args: TensorInterface, **extra_kwargs) -> ProgramData:
        raise NotImplementedError()

    def cache_policy(self, *args: TensorInterface, **extra_kwargs) -> Hashable:
        return tuple((x.shape, x.strides, x.typechr, x.elm_size) for x in args) + tuple(sorted(extra_kwargs.items()))

    def executor_warp_size(self) -> int:
        return get_executor().warp_size()

    def __call__(self, *args, grid_dim: int, **extra_kwargs):
        # Calling a gint program from inside a torch.compile trace must not be traced: run it as a graph break.
        if torch.compiler.is_compiling():
            return _call_untraced(self, args, grid_dim, extra_kwargs)
        get_executor().execute(self, [_convert_arg(a) for a in args], grid_dim, **extra_kwargs)


@torch.compiler.disable
def _call_untraced(program, args, grid_dim, extra_kwargs):
    get_executor().execute(program, [_convert_arg(a) for a in args], grid_dim, **extra_kwargs)


class BaseExecutor:
    def warp_size(self) -> int:
        raise NotImplementedError

    def execute(self, program: BaseExecutableProgram, args: Sequence[TensorInterface], grid_dim: int, **extra_kwargs):
        raise NotImplementedError

    def execute_indirect(self, programs: Sequence[BaseExecutableProgram], args_list: Sequence[Sequence[TensorInterface]],
                         indices: Sequence[int], **extra_kwargs):
        raise NotImplementedError


class _Cacheline:
    __slots__ = ("handle", "indices", "ptrs", "n", "pd")

    def __init__(self, handle, indices, pd):
        self.handle = handle
        self.indices = indices
        self.n = len(indices)
        self.ptrs = (ctypes.c_uint64 * MAX_N_TENSORS)()
        self.pd = pd


class B200Executor(BaseExecutor):
    """Launches gint programs through libgint_b200.so. One library context per CUDA device, created on first use."""

    def __init__(self) -> None:
        self._lib = capi.load_library()
        self._ctxs: dict[int, ctypes.c_void_p] = {}
        self._lock = threading.Lock()
        self.launches = 0          # number of kernel launches issued through this executor
        self._copy_streams: dict[int, tuple] = {}   # per device: (host-to-device, device-to-host) copy streams

    # ------------------------------------------------------------------ plumbing
    def warp_size(self) -> int:
        return 32

    def _ctx(self, device: Optional[int] = None):
        if device is None:
            device = torch.cuda.current_device()
        ctx = self._ctxs.get(device)
        if ctx is None:
            with self._lock:
                ctx = self._ctxs.get(device)
                if ctx is None:
                    if not torch.cuda.is_available():
                        raise capi.GintError(capi.GINT_ERR_NO_DEVICE, "CUDA is not available; gint_b200 has no CPU path")
                    torch.cuda.init()
                    out = ctypes.c_void_p()
                    rc = self._lib.gint_create(device, ctypes.byref(out))
                    if rc != 0:
                        raise capi.GintError(rc, f"gint_create(device={device}): {capi.status_string(rc)}")
                    ctx = self._ctxs[device] = out
        return device, ctx

    def _check(self, ctx, rc: int, what: str):
        if rc == 0:
            return
        msg = self._lib.gint_last_error(ctx).decode(errors="replace")
        if rc == capi.GINT_ERR_ARG_COUNT:
            raise ValueError("Number of arguments don't match the program.")
        if rc in (capi.GINT_ERR_UNKNOWN_OPCODE, capi.GINT_ERR_STACK_UNDERFLOW, capi.GINT_ERR_STACK_OVERFLOW, capi.GINT_ERR_NO_HALT):
            raise ValueError(f"{what}: {msg}")
        raise capi.GintError(rc, f"{what}: {msg}")

    def _build_cacheline(self, ctx, program, args, extra_kwargs) -> _Cacheline:
        pd = program.get_program(*args, **extra_kwargs)
        if pd.input_indices is None:
            pd.input_indices = list(range(len(pd.input_infos)))
        if len(pd.input_indices) != len(pd.input_infos):
            raise AssertionError("Input indices must match input infos")
        if len(args) != len(pd.input_indices):
            raise ValueError("Number of arguments don't match the program.")
        if len(pd.input_infos) > MAX_N_TENSORS:
            raise ValueError(f"At most {MAX_N_TENSORS} tensors per program")
        pd.stats  # raises ValueError on unknown opcodes / stack underflow, like the reference's select_variant
        code = numpy.ascontiguousarray(numpy.asarray(pd.program, dtype=numpy.int32).reshape(-1))
        ti = capi.HTensorInfo()
        fill_tensor_info(ti, pd.input_infos)
        handle = ctypes.c_uint64()
        rc = self._lib.gint_program_create(ctx, code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size),
                                           ctypes.byref(ti), len(pd.input_infos), ctypes.byref(handle))
        self._check(ctx, rc, "gint_program_create")
        return _Cacheline(handle.value, list(pd.input_indices), pd)

    def _cacheline(self, program, args, extra_kwargs):
        device, ctx = self._ctx()
        cache = program.__dict__.get("_b200")
        if cache is None:
            cache = program._b200 = {}
        key = (device, program.cache_policy(*args, **extra_kwargs))
        line = cache.get(key)
        if line is None:
            line = cache[key] = self._build_cacheline(ctx, program, args, extra_kwargs)
        return ctx, line

    # ------------------------------------------------------------------ BaseExecutor API
    def execute(self, program: BaseExecutableProgram, args: Sequence[TensorInterface], grid_dim: int, cuda_stream: int = 0,
                **extra_kwargs):
        ctx, line = self._cacheline(program, args, extra_kwargs)
        ptrs = line.ptrs
        for i, a in enumerate(line.indices):
            ptrs[i] = args[a].base_ptr
        rc = self._lib.gint_execute(ctx, line.handle, ptrs, line.n, grid_dim, cuda_stream)
        if rc != 0:
            self._check(ctx, rc, "gint_execute")
        self.launches += 1

    def execute_gathered(self, program: BaseExecutableProgram, args: Sequence[TensorInterface], grid_dim: int, gathered: Sequence[int],
                         row_index, cuda_stream: int = 0, **extra_kwargs):
        """``execute`` in which the arguments listed in ``gathered`` (argument indices) are TABLES read through ``row_index``:
        logical program b works on row ``row_index[b]`` of such a tensor instead of row b (its descriptor's innermost batch
        dimension). ``row_index`` is an int64 device tensor. ``table[index]`` feeds the program without a gather kernel and an
        intermediate copy (``gint_execute_gathered``)."""
        ctx, line = self._cacheline(program, args, extra_kwargs)
        ptrs = line.ptrs
        mask, extent, rows = 0, 0, 0
        for i, a in enumerate(line.indices):
            ptrs[i] = args[a].base_ptr
            if a in gathered:
                mask |= 1 << i
                t = args[a]
                extent = max(extent, (sum((s - 1) * abs(st) for s, st in zip(t.shape, t.strides) if s > 0) + 1) * t.elm_size)
                if rows and rows != t.shape[0]:
                    raise ValueError("gathered tables of one launch must have the same number of rows")
                rows = t.shape[0]
        rc = self._lib.gint_execute_gathered(ctx, line.handle, ptrs, line.n, grid_dim, mask, ctypes.c_void_p(row_index.data_ptr()), rows, extent,
                                             cuda_stream)
        if rc != 0:
            self._check(ctx, rc, "gint_execute_gathered")
        self.launches += 1

    def execute_checked(self, program: BaseExecutableProgram, args: Sequence[TensorInterface], grid_dim: int, cuda_stream: int = 0,
                        **extra_kwargs):
        """``execute`` on the bounds-checking kernel (``gint_execute_checked``): every access is compared with the byte range
        of the tensor VIEW that was passed (base pointer, shape and strides of its ``TensorInterface``); an access outside it
        is skipped and recorded. Read the outcome with ``device_status()``. For developing programs and descriptors; slow."""
        ctx, line = self._cacheline(program, args, extra_kwargs)
        n = line.n
        ptrs, lo, hi = line.ptrs, (ctypes.c_uint64 * MAX_N_TENSORS)(), (ctypes.c_uint64 * MAX_N_TENSORS)()
        for i, a in enumerate(line.indices):
            t = args[a]
            ptrs[i] = t.base_ptr
            below = sum(min(0, (s - 1) * st) for s, st in zip(t.shape, t.strides) if s > 0)
            above = sum(max(0, (s - 1) * st) for s, st in zip(t.shape, t.strides) if s > 0)
            empty = any(s == 0 for s in t.shape)
            lo[i] = t.base_ptr + below * t.elm_size
            hi[i] = lo[i] if empty else t.base_ptr + (above + 1) * t.elm_size
        rc = self._lib.gint_execute_checked(ctx, line.handle, ptrs, lo, hi, n, grid_dim, cuda_stream)
        if rc != 0:
            self._check(ctx, rc, "gint_execute_checked")
        self.launches += 1

    def device_status(self, clear: bool = True, device: Optional[int] = None) -> dict:
        """What the checked launches on ``device`` found so far (waits for the device): ``code`` 0 means nothing; otherwise
        the first event's kind, tensor slot, logical program, instruction index, address and lane, and the event count."""
        _, ctx = self._ctx(device)
        st = capi.DeviceStatusC()
        rc = self._lib.gint_device_status_read(ctx, ctypes.byref(st), 1 if clear else 0)
        self._check(ctx, rc, "gint_device_status_read")
        out = {name: getattr(st, name) for name, _ in capi.DeviceStatusC._fields_}
        out["what"] = capi.DEVICE_CODES.get(st.code, "unknown")
        return out

    def execute_range(self, program: BaseExecutableProgram, args: Sequence[TensorInterface], first: int, count: int,
                      cuda_stream: int = 0, **extra_kwargs):
        """Run logical programs ``[first, first + count)`` of the program's grid (multi-GPU sharding primitive)."""
        ctx, line = self._cacheline(program, args, extra_kwargs)
        ptrs = line.ptrs
        for i, a in enumerate(line.indices):
            ptrs[i] = args[a].base_ptr
        rc = self._lib.gint_execute_range(ctx, line.handle, ptrs, line.n, first, count, cuda_stream)
        if rc != 0:
            self._check(ctx, rc, "gint_execute_range")
        self.launches += 1

    def execute_indirect(self, programs: Sequence[BaseExecutableProgram], args_list: Sequence[Sequence], indices: Sequence[int],
                         cuda_stream: int = 0, static_tables: bool = False):
        """One launch; logical program ``i`` runs ``programs[indices[i]]`` on ``args_list[indices[i]]``
        (``gint/host/cuda/executor_impl.py:135-201``).

        ``static_tables=True`` routes the launch through ``gint_execute_indirect_static``: the same kernel and results, but
        the per-launch tables go into a fixed array inside the library instead of scratch memory that may be (re)allocated,
        for callers that must not allocate device memory at launch time. At most 64 programs and 4096 logical programs;
        the first such call on a device does a one-time set-up that synchronises the device."""
        if len(programs) != len(args_list):
            raise AssertionError("programs and args_list must have the same length")
        n = len(programs)
        grid_dim = len(indices)
        if n == 0 or grid_dim == 0:
            return
        handles = (ctypes.c_uint64 * n)()
        ptrs = (ctypes.c_uint64 * (n * MAX_N_TENSORS))()
        ctx = None
        for p, (prog, args) in enumerate(zip(programs, args_list)):
            conv = [_convert_arg(a) for a in args]
            c, line = self._cacheline(prog, conv, {})
            if ctx is not None and c is not ctx and c.value != ctx.value:
                raise ValueError("execute_indirect: the programs of one launch must live on one device")
            ctx = c
            handles[p] = line.handle
            for i, a in enumerate(line.indices):
                ptrs[p * MAX_N_TENSORS + i] = conv[a].base_ptr
        idx = (ctypes.c_int32 * grid_dim)(*[int(i) for i in indices])
        fn = self._lib.gint_execute_indirect_static if static_tables else self._lib.gint_execute_indirect
        rc = fn(ctx, handles, n, ptrs, idx, grid_dim, cuda_stream)
        if rc != 0:
            self._check(ctx, rc, "gint_execute_indirect_static" if static_tables else "gint_execute_indirect")
        self.launches += 1

    def build_plan(self, steps: Sequence[tuple]) -> "Plan":
        """Lower a list of ``(program, args, grid_dim)`` steps -- what a compiled graph is after the conductor has run --
        into one reusable ``Plan``: programs are built (or found in their caches) now, the tensor addresses are written
        into a C array, and ``Plan.run(cuda_stream)`` launches every step with a single library call
        (``gint_execute_plan``). Replaces the Python loop of the conductor's ``execute`` closure
        (``gint/conductor/compiler.py:1442-1485``). ``Plan.set_arg`` re-points one argument of one step (fresh
        input / output tensors per call)."""
        plan_steps = (capi.PlanStepC * len(steps))()
        ctx = None
        slots = []
        for i, (program, args, grid_dim) in enumerate(steps):
            conv = [_convert_arg(a) for a in args]
            ctx, line = self._cacheline(program, conv, {})
            plan_steps[i].handle = line.handle
            plan_steps[i].n_tensors = line.n
            plan_steps[i].grid_dim = grid_dim
            for j, a in enumerate(line.indices):
                plan_steps[i].base_ptrs[j] = conv[a].base_ptr
            slots.append(list(line.indices))
        return Plan(self, ctx, plan_steps, slots)

    def execute_streamed(self, program: BaseExecutableProgram, args: Sequence[torch.Tensor], grid_dim: int,
                         host_inputs: dict, host_outputs: dict, n_chunks: int = 16, **extra_kwargs):
        """Run ``program`` on data that lives in HOST memory, overlapping the transfers with the kernels.

        ``args`` are the device tensors the program works on (one per argument, as for ``execute``); ``host_inputs`` maps
        argument indices to (pinned) host tensors that are copied into those device tensors first, ``host_outputs`` maps
        argument indices to (pinned) host tensors that receive the results. The logical grid is cut into ``n_chunks``
        contiguous ranges; range c is copied in on one copy stream, run with ``gint_execute_range`` on the current stream
        and copied out on a second copy stream, so the host-to-device copy of range c+1, the kernel of range c and the
        device-to-host copy of range c-1 proceed at the same time (the two directions of the link are independent). A
        tensor is cut along with the grid when the descriptor decode places logical program i at i times a fixed offset
        from the base pointer (the rule of ``gint_b200.shard.element_offset``); any other tensor (broadcast operands,
        irregular layouts) is copied whole, inputs before the first range and outputs after the last. On return the
        current stream waits for the last copy. No counterpart in the reference, which takes device tensors only."""
        from ..shard import element_offset, shard_range
        device, _ = self._ctx()
        conv = [_convert_arg(a) for a in args]
        ctx, line = self._cacheline(program, conv, extra_kwargs)
        infos = line.pd.input_infos

        code = numpy.asarray(line.pd.program, dtype=numpy.int64).reshape(-1, 2)

        def reach(slot: int):
            """Upper bound (elements) on how far from its tile's first element a logical program reaches into slot `slot`,
            ignoring the shape masks; None if it cannot be bounded (gather/scatter, moving base)."""
            from .. import opcodes as O
            info = infos[slot]
            s1, s2 = abs(info.block_shape_stride_1[1]), abs(info.block_shape_stride_2[1])
            far = 0
            for op, operand in code:
                op, operand = int(op), int(operand) & 0xFFFFFFFF
                name = O.NAMES[op] if 0 <= op < len(O.NAMES) else ""
                if not (name.startswith("LoadGlobal") or name.startswith("StoreGlobal") or name.startswith("Advance")) or (operand & 15) != slot:
                    continue
                if name.startswith("Advance") or name.endswith("Indirect"):
                    return None
                off = operand >> 4
                if "1D" in name:
                    far = max(far, (off + 127) * s1)
                else:   # 32 rows or columns of four values
                    far = max(far, 31 * s1 + (off + 3) * s2, (off + 3) * s1 + 31 * s2)
            return far

        def cut(arg_index: int):
            """bytes per logical program if the tensor can be cut along the grid (logical program i touches only bytes
            [i*step, (i+1)*step) of it), else None"""
            slots = [i for i, a in enumerate(line.indices) if a == arg_index]
            if not slots:
                return None
            steps = set()
            for i in slots:
                if infos[i].block_shape_stride_1[1] < 0 or infos[i].block_shape_stride_2[1] < 0:
                    return None
                one = element_offset(infos[i], 1)
                probes = {grid_dim - 1, grid_dim // 2, 2}
                if one == 0 or any(element_offset(infos[i], k) != k * one for k in probes if 0 <= k < grid_dim):
                    return None
                far = reach(i)
                if far is None or far >= one:
                    return None
                steps.add(one * infos[i].elm_size)
            return steps.pop() if len(steps) == 1 else None

        def as_bytes(t: torch.Tensor) -> torch.Tensor:
            return t.contiguous().view(torch.uint8).reshape(-1) if not t.is_contiguous() else t.view(torch.uint8).reshape(-1)

        plan = []   # (device bytes, host bytes, bytes per logical program or None, is_input)
        for table, is_input in ((host_inputs, True), (host_outputs, False)):
            for a, host in table.items():
                dev = args[a]
                if not (dev.is_contiguous() and host.is_contiguous()) or dev.numel() * dev.element_size() != host.numel() * host.element_size():
                    raise ValueError("execute_streamed needs contiguous host and device tensors of equal size")
                plan.append((as_bytes(dev), as_bytes(host), cut(a), is_input))
        streams = self._copy_streams.get(device)
        if streams is None:
            streams = self._copy_streams[device] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        h2d, d2h = streams
        compute = torch.cuda.current_stream(device)
        start = torch.cuda.Event()
        start.record(compute)
        h2d.wait_event(start)
        d2h.wait_event(start)
        with torch.cuda.stream(h2d):
            for dev, host, step, is_input in plan:
                if is_input and step is None:
                    dev.copy_(host, non_blocking=True)
        n_chunks = max(1, min(int(n_chunks), grid_dim))
        for c in range(n_chunks):
            first, count = shard_range(grid_dim, n_chunks, c)
            last = c == n_chunks - 1
            with torch.cuda.stream(h2d):
                for dev, host, step, is_input in plan:
                    if is_input and step is not None:
                        lo, hi = first * step, (dev.numel() if last else min((first + count) * step, dev.numel()))
                        if lo < hi:
                            dev[lo:hi].copy_(host[lo:hi], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(h2d)
            compute.wait_event(arrived)
            self.execute_range(program, conv, first, count, cuda_stream=compute.cuda_stream, **extra_kwargs)
            computed = torch.cuda.Event()
            computed.record(compute)
            with torch.cuda.stream(d2h):
                d2h.wait_event(computed)
                for dev, host, step, is_input in plan:
                    if not is_input and (step is not None or last):
                        lo, hi = (0, dev.numel()) if step is None else (first * step, dev.numel() if last else min((first + count) * step, dev.numel()))
                        if lo < hi:
                            host[lo:hi].copy_(dev[lo:hi], non_blocking=True)
        done = torch.cuda.Event()
        done.record(d2h)
        compute.wait_event(done)

    # ------------------------------------------------------------------ introspection / tuning
    def launch_info(self, program: BaseExecutableProgram, args: Sequence, grid_dim: int, **extra_kwargs) -> dict:
        args = [_convert_arg(a) for a in args]
        ctx, line = self._cacheline(program, args, extra_kwargs)
        info = capi.LaunchInfoC()
        rc = self._lib.gint_program_launch_info(ctx, line.handle, grid_dim, ctypes.byref(info))
        self._check(ctx, rc, "gint_program_launch_info")
        return {name: getattr(info, name) for name, _ in capi.LaunchInfoC._fields_ if name != "reserved"}

    def set_option(self, name: str, value: int, device: Optional[int] = None) -> None:
        _, ctx = self._ctx(device)
        rc = self._lib.gint_set_option(ctx, name.encode(), int(value))
        self._check(ctx, rc, f"gint_set_option({name})")

    def close(self) -> None:
        for ctx in self._ctxs.values():
            self._lib.gint_destroy(ctx)
        self._ctxs.clear()


class Plan:
    """A lowered list of launches (see ``B200Executor.build_plan``). Valid on the device it was built on, for as long as
    the programs live; the tensors whose addresses it holds must outlive every ``run``."""

    def __init__(self, owner: "B200Executor", ctx, steps, slots) -> None:
        self._owner, self._ctx, self._steps, self._slots = owner, ctx, steps, slots
        self._n = len(steps)
        self._n_launches = sum(1 for s in steps if s.grid_dim)
        self._call = owner._lib.gint_execute_plan

    def __len__(self) -> int:
        return self._n

    def set_arg(self, step: int, arg_index: int, tensor) -> None:
        """Point argument ``arg_index`` of step ``step`` at another tensor of the same shape and strides."""
        ptr = _convert_arg(tensor).base_ptr
        for j, a in enumerate(self._slots[step]):
            if a == arg_index:
                self._steps[step].base_ptrs[j] = ptr

    def run(self, cuda_stream: int = 0) -> None:
        if self._n == 0:
            return
        rc = self._call(self._ctx, self._steps, self._n, cuda_stream)
        if rc != 0:
            self._owner._check(self._ctx, rc, "gint_execute_plan")
        self._owner.launches += self._n_launches


executor: Optional[BaseExecutor] = None


def get_executor() -> BaseExecutor:
    """The process-wide executor (``gint/host/executor.py:212-233``); always the B200 one here."""
    global executor
    if executor is None:
        executor = B200Executor()
    return executor


def c_analyze(program) -> dict:
    """Run the library's own static analysis (``gint_analyze``) on a bytecode array; no GPU needed."""
    lib = capi.load_library()
    code = numpy.ascontiguousarray(numpy.asarray(program, dtype=numpy.int32).reshape(-1))
    st = capi.BytecodeStatsC()
    rc = lib.gint_analyze(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size), ctypes.byref(st))
    out = {name: getattr(st, name) for name, _ in capi.BytecodeStatsC._fields_ if name != "reserved"}
    out["status"] = rc
    return out
