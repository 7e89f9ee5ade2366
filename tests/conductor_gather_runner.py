#!/usr/bin/env python
"""Child process of tests/test_gpu_conductor_gather.py: the benchmark's conductor graph (configs[4], written with F.silu) through
``torch.compile(backend="gint")`` of the reference package in ``baseline/_ref``, with the B200 executor and its conductor fast
path installed. Prints one JSON object."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.join(ROOT, "tests")]
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

torch.zeros(1, device="cuda")
import gint_b200  # noqa: E402
from gint_b200 import conductor_fastpath  # noqa: E402

ex = gint_b200.install(accelerate_conductor=True)
import gint.conductor  # noqa: E402,F401  (registers the backend)


def graph(x, idx, w):
    g = x[idx]
    y = g * torch.rsqrt(torch.mean(g * g, dim=-1, keepdim=True) + 1e-6) * w
    z = F.silu(y) + x
    return z, z.sum(-1)


out = {}
gen = torch.Generator().manual_seed(42)
R, N = 2048, 1024
x = torch.randn(R, N, generator=gen).cuda()
w = (1.0 + 0.1 * torch.randn(N, generator=gen)).cuda()
cases = {"positive": torch.randint(0, R, (R,), generator=gen).cuda(),
         "negative": (torch.randint(0, R, (R,), generator=gen) - R).cuda(),       # counts from the end, as torch does
         "int32": torch.randint(0, R, (R,), generator=gen).to(torch.int32).cuda()}  # not foldable: falls back to torch's gather
for name, idx in cases.items():
    torch._dynamo.reset()
    n_before = len(conductor_fastpath.ACCELERATED)
    fn = torch.compile(graph, backend="gint", options={"cuda_graphs": False})
    with torch.no_grad():
        z_ref, s_ref = graph(x, idx.long() if idx.dtype != torch.int64 else idx, w)
        fn(x, idx, w)                      # compile + first run
        launches = ex.launches
        z, s = fn(x, idx, w)
        torch.cuda.synchronize()
    closures = conductor_fastpath.ACCELERATED[n_before:]
    out[name] = {"launches_per_call": ex.launches - launches, "closures": len(closures),
                 "foldable": sum(getattr(c, "foldable_gathers", 0) for c in closures), "folded": sum(getattr(c, "gathers_folded", 0) for c in closures),
                 "z_max_abs_err": float((z - z_ref).abs().max()), "s_max_rel_err": float(((s - s_ref).abs() / s_ref.abs().clamp_min(1.0)).max()),
                 "z_close": bool(torch.allclose(z, z_ref, rtol=1e-5, atol=1e-5)), "s_close": bool(torch.allclose(s, s_ref, rtol=1e-4, atol=1e-3))}
# the two programs the live conductor emitted are the recorded ones (gint_b200/data/programs.json, made from the same graph
# with FakeTensors): same instruction streams; the descriptors differ only in the number of rows
import numpy as np  # noqa: E402
from gint_b200.programs import recorded  # noqa: E402
live = []
for c in conductor_fastpath.ACCELERATED:
    env = conductor_fastpath._closure_vars(getattr(c, "original", c))
    for entry in env.get("sg_dispatch", []):
        live.append(np.asarray(entry[0].bytecode, dtype=np.int32).reshape(-1))
want = [recorded("graph_fused_r65536_n1024").bytecode, recorded("graph_rowsum_r65536_n1024").bytecode]
out["programs_equal_recorded"] = all(any(a.shape == b.shape and bool((a == b).all()) for a in live) for b in want)
out["live_program_lengths"] = sorted({int(a.size // 2) for a in live})
print(json.dumps(out))
