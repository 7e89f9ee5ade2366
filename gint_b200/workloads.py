"""The five named bytecode programs with seeded synthetic inputs, their torch-eager expressions and byte counts.

Each workload pairs recorded bytecode (``gint_b200.programs``) with:

* ``make_inputs``: the synthetic inputs of the benchmark definition, generated on the CPU from a seed so the CPU and
  GPU sides see identical bits, then moved to the requested device;
* ``eager``: the torch-eager expression the reference's own tests compare against
  (``tests/test_a_plus_b_executor.py:87``, ``tests/test_conductor_backend.py:546-596``, ``tests/test_bmm4x4.py:50``,
  ``tests/test_inv4x4.py:233``) -- used as the oracle of last resort and as the timed CPU baseline;
* ``algorithmic_bytes``: bytes that must cross HBM once (inputs read once + outputs written once).

``leading`` is the size of the independent leading dimension (elements, rows or matrices). A multi-GPU run gives each
rank ``leading / world`` of it; recorded programs exist for the full size and for 1/2, 1/4 and 1/8 of it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .programs import RecordedProgram, recorded


@dataclass
class Step:
    program: RecordedProgram
    roles: list[str]          # tensor role for each program argument
    grid_dim: int
    gathered: tuple = ()      # argument positions that are tables read through `row_index` (B200Executor.execute_gathered)
    row_index: str = ""       # role of the int64 row-index tensor


@dataclass
class Workload:
    name: str
    config: str               # which benchmark configuration this is
    leading: int
    inner: int
    tensors: dict = field(default_factory=dict)      # role -> tensor
    steps: list = field(default_factory=list)
    outputs: list = field(default_factory=list)       # roles written by the program(s)
    pre: Optional[Callable] = None                    # eager work the reference also leaves outside the interpreter
    elements: int = 0
    algorithmic_bytes: int = 0
    rtol: float = 1e-5
    atol: float = 1e-6
    _args_cache: Optional[tuple] = field(default=None, repr=False, compare=False)

    def run(self, executor, stream: int = 0) -> None:
        if self.pre is not None:
            self.pre(self.tensors)
        for st, args in zip(self.steps, self._interfaces()):
            if st.gathered:
                executor.execute_gathered(st.program, args, st.grid_dim, st.gathered, self.tensors[st.row_index], cuda_stream=stream)
            else:
                executor.execute(st.program, args, st.grid_dim, cuda_stream=stream)

    def _interfaces(self):
        """The steps' arguments as TensorInterfaces, converted once (a caller that launches the same tensors again and again
        keeps the converted form; the conductor's compiled graphs do the same with their skeletons)."""
        from .host.executor import _convert_arg
        key = tuple(t.data_ptr() for t in self.tensors.values())
        if self._args_cache is None or self._args_cache[0] != key:
            self._args_cache = (key, [[_convert_arg(self.tensors[r]) for r in st.roles] for st in self.steps])
        return self._args_cache[1]

    def plan(self, executor):
        """The bytecode steps as one reusable launch plan (``B200Executor.build_plan``); ``pre`` stays with the caller. None for a
        workload with gathered rows (plans carry plain launches only)."""
        if any(st.gathered for st in self.steps):
            return None
        return executor.build_plan([(st.program, [self.tensors[r] for r in st.roles], st.grid_dim) for st in self.steps])

    def launches_per_run(self) -> int:
        return len(self.steps)


def _rand(gen, *shape):
    return torch.rand(*shape, generator=gen, dtype=torch.float32)


def _randn(gen, *shape):
    return torch.randn(*shape, generator=gen, dtype=torch.float32)


# ---------------------------------------------------------------------------------------------- eager expressions

def eager_add(t):
    return {"out": t["a"] + t["b"]}


def eager_rmsnorm(t, eps: float = 1e-6):
    x, w = t["x"], t["w"]
    return {"out": x * torch.rsqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps) * w}


def eager_bmm(t):
    B = t["a"].shape[0]
    return {"c": torch.bmm(t["a"].view(B, 4, 4), t["b"].view(B, 4, 4)).reshape(B, 16)}


def eager_inv(t):
    B = t["a"].shape[0]
    return {"c": torch.linalg.inv(t["a"].view(B, 4, 4)).reshape(B, 16)}


def eager_graph(t, eps: float = 1e-6):
    g = t["x_full"][t["idx"]]
    y = g * torch.rsqrt(torch.mean(g * g, dim=-1, keepdim=True) + eps) * t["w"]
    z = F.silu(y) + t["x_rows"]
    return {"z": z, "s": z.sum(-1)}


EAGER = {"add": eager_add, "rmsnorm": eager_rmsnorm, "bmm4x4": eager_bmm, "inv4x4": eager_inv, "graph": eager_graph, "graph_gathered": eager_graph}

FULL_SIZES = {"add": (1048576, 1), "rmsnorm": (16384, 4096), "bmm4x4": (4194304, 16), "inv4x4": (4194304, 16),
              "graph": (65536, 1024), "graph_gathered": (65536, 1024)}
GRAPH_TABLE_ROWS = 65536   # x_full of the conductor graph; replicated on every GPU because x_full[idx] reads any row


# ---------------------------------------------------------------------------------------------- builders

def make_workload(name: str, leading: Optional[int] = None, inner: Optional[int] = None, device="cuda", seed: int = 42,
                  table_rows: Optional[int] = None) -> Workload:
    """Build a workload on `device`. Sizes default to the full benchmark configuration; other sizes must have a
    recorded program (see tests/golden/make_golden.py for the list)."""
    full_leading, full_inner = FULL_SIZES[name]
    leading = full_leading if leading is None else leading
    inner = full_inner if inner is None else inner
    gen = torch.Generator().manual_seed(seed)
    dev = torch.device(device)

    if name == "add":
        prog = recorded(f"add_n{leading}")
        t = {"a": _randn(gen, leading), "b": _randn(gen, leading), "out": torch.zeros(leading)}
        wl = Workload("add", "configs[0]: a+b elementwise add", leading, 1, steps=[Step(prog, prog.arg_roles, prog.grid_dim)],
                      outputs=["out"], elements=leading, algorithmic_bytes=12 * leading)
    elif name == "rmsnorm":
        prog = recorded(f"rmsnorm_r{leading}_n{inner}")
        t = {"x": _randn(gen, leading, inner), "w": 1.0 + 0.1 * _randn(gen, inner), "out": torch.zeros(leading, inner)}
        wl = Workload("rmsnorm", "configs[1]: RMSNorm over rows", leading, inner, steps=[Step(prog, prog.arg_roles, prog.grid_dim)],
                      outputs=["out"], elements=leading * inner, algorithmic_bytes=2 * 4 * leading * inner + 4 * inner)
    elif name == "bmm4x4":
        prog = recorded(f"bmm4x4_b{leading}")
        t = {"a": _rand(gen, leading, 16) * 2 - 1, "b": _rand(gen, leading, 16) * 2 - 1, "c": torch.zeros(leading, 16)}
        wl = Workload("bmm4x4", "configs[2]: batched 4x4 matmul", leading, 16, steps=[Step(prog, prog.arg_roles, prog.grid_dim)],
                      outputs=["c"], elements=leading * 16, algorithmic_bytes=3 * 64 * leading)
    elif name == "inv4x4":
        prog = recorded(f"inv4x4_b{leading}")
        a = (_rand(gen, leading, 4, 4) * 2 - 1) + 4.0 * torch.eye(4)
        t = {"a": a.reshape(leading, 16).contiguous(), "c": torch.zeros(leading, 16)}
        wl = Workload("inv4x4", "configs[3]: batched 4x4 inverse", leading, 16, steps=[Step(prog, prog.arg_roles, prog.grid_dim)],
                      outputs=["c"], elements=leading * 16, algorithmic_bytes=2 * 64 * leading, rtol=1e-4, atol=1e-4)
    elif name in ("graph", "graph_gathered"):
        fused = recorded(f"graph_fused_r{leading}_n{inner}")
        rowsum = recorded(f"graph_rowsum_r{leading}_n{inner}")
        table = table_rows or (GRAPH_TABLE_ROWS if inner == 1024 and leading >= 8192 else {96: 128, 10: 16}.get(leading, leading))
        x_full = _randn(gen, table, inner)
        idx = torch.randint(0, table, (leading,), generator=gen, dtype=torch.int64)
        w = 1.0 + 0.1 * _randn(gen, inner)
        # residual rows: the first `leading` rows of the table (the whole table at full size)
        t = {"x_full": x_full, "x_rows": x_full[:leading], "idx": idx, "w": w, "g": torch.zeros(leading, inner),
             "z": torch.zeros(leading, inner), "s": torch.zeros(leading)}

        def gather(tt):
            # aten.index.Tensor stays a torch kernel in the reference too (not lowered by the conductor)
            torch.index_select(tt["x_full"], 0, tt["idx"], out=tt["g"])
        row = 4 * inner
        wl = Workload("graph", "configs[4]: conductor graph (gather + rmsnorm + silu + residual, row sum)", leading, inner,
                      steps=[Step(fused, fused.arg_roles, fused.grid_dim), Step(rowsum, rowsum.arg_roles, rowsum.grid_dim)],
                      outputs=["z", "s"], pre=gather, elements=leading * inner,
                      # as executed (3 kernels): gather R+W, fused R(g)+R(x)+W(z), sum R(z); plus idx, w, s
                      algorithmic_bytes=leading * row * 6 + leading * 8 + 4 * inner + 4 * leading)
        if name == "graph_gathered":
            # the same two bytecode programs, but the fused one reads x_full[idx] in place: its `g` argument is the table and
            # logical program b works on row idx[b] (gint_execute_gathered) -- no gather kernel, no intermediate g
            g_pos = fused.arg_roles.index("g")
            roles = [("x_full" if r == "g" else r) for r in fused.arg_roles]
            wl = Workload("graph_gathered", "configs[4] with the gather folded into the fused program's row loads (2 kernels)", leading, inner,
                          steps=[Step(fused, roles, fused.grid_dim, gathered=(g_pos,), row_index="idx"), Step(rowsum, rowsum.arg_roles, rowsum.grid_dim)],
                          outputs=["z", "s"], pre=None, elements=leading * inner,
                          # R(x_full[idx]) + R(x_rows) + W(z); sum R(z); plus idx, w, s
                          algorithmic_bytes=leading * row * 4 + leading * 8 + 4 * inner + 4 * leading)
    else:
        raise KeyError(name)

    wl.tensors = {k: v.to(dev) for k, v in t.items()}
    if name in ("graph", "graph_gathered"):
        # keep x_rows a view of the table on the device as well
        wl.tensors["x_rows"] = wl.tensors["x_full"][:leading]
    return wl


def check_outputs(wl: Workload, reference: dict, rtol: Optional[float] = None, atol: Optional[float] = None) -> dict:
    """Compare the workload's output tensors with `reference` (role -> tensor); returns max abs error per output."""
    errs = {}
    for role in wl.outputs:
        got = wl.tensors[role].detach().cpu()
        ref = reference[role].detach().cpu()
        torch.testing.assert_close(got, ref.reshape(got.shape), rtol=wl.rtol if rtol is None else rtol,
                                   atol=wl.atol if atol is None else atol)
        errs[role] = float((got - ref.reshape(got.shape)).abs().max())
    return errs
