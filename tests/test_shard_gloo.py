"""Multi-rank host logic on CPU (world_size 2 and 3, gloo): shard planning, pointer biasing and result assembly.

Each rank plans its shard of a full-size recorded program (gint_b200.shard), runs ONLY its range of the logical grid on
rank-local buffers through the CPU oracle (standing in for its GPU), and the shards are gathered with gloo and compared,
bit for bit, with the unsharded run. No collective is part of the data path: the all_gather here is the test's check.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gint_b200.shard import element_offset, plan_shard, shard_range
from gint_b200.workloads import make_workload
from oracle import oracle


def test_shard_range_is_a_partition():
    for grid in (0, 1, 7, 64, 16384, 131072):
        for world in (1, 2, 3, 8):
            spans = [shard_range(grid, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == grid
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f0 + c0 == f1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1


def test_element_offset_matches_row_layouts():
    wl = make_workload("rmsnorm", 64, 4096, device="cpu")
    infos = {r: t for r, t in zip(wl.steps[0].roles, wl.steps[0].program.tensor_infos)}
    assert [element_offset(infos["x"], i) for i in (0, 1, 33)] == [0, 4096, 33 * 4096]
    assert [element_offset(infos["w"], i) for i in (0, 1, 33)] == [0, 0, 0]          # broadcast operand: replicated
    wl = make_workload("bmm4x4", 1000, 16, device="cpu")
    a = wl.steps[0].program.tensor_infos[0]
    assert [element_offset(a, i) for i in (0, 1, 5)] == [0, 32 * 16, 5 * 32 * 16]    # 32 matrices of 16 floats per logical program


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, name: str, leading: int, inner: int, out_path: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        full = make_workload(name, leading, inner, device="cpu")        # same seed on every rank: identical inputs
        st = full.steps[0]
        infos = st.program.tensor_infos
        plan = plan_shard(infos, st.grid_dim, world, rank)
        # rank-local buffers: the slice of every sharded tensor that this rank's logical programs touch
        local, ptrs = {}, []
        next_first = plan.first + plan.count
        for role, info, bias in zip(st.roles, infos, plan.byte_bias):
            t = full.tensors[role]
            flat = t.reshape(-1)
            if element_offset(info, 1 if st.grid_dim > 1 else 0) == 0 and bias == 0 and element_offset(info, st.grid_dim - 1) == 0:
                local[role] = flat.clone()                                 # replicated operand
            else:
                lo = bias // info.elm_size
                hi = element_offset(info, next_first) if next_first < st.grid_dim else flat.numel()
                local[role] = flat[lo:hi].clone()
            ptrs.append(local[role].data_ptr())
        oracle.execute_range(st.program.bytecode, [vars(t) for t in infos], plan.biased(ptrs), plan.first, plan.count)
        # gather the output shards (variable length -> gather objects) and assemble on rank 0
        out_role = full.outputs[0]
        pieces = [None] * world
        dist.all_gather_object(pieces, (plan.first, local[out_role]))
        times = torch.tensor([float(rank + 1)])
        dist.all_reduce(times, op=dist.ReduceOp.MAX)                        # the bench's max-over-ranks reduction
        assert times.item() == float(world)
        if rank == 0:
            oracle.execute(st.program.bytecode, [vars(t) for t in infos], [full.tensors[r] for r in st.roles], st.grid_dim,
                           input_indices=st.program.input_indices)
            got = torch.cat([p for _, p in sorted(pieces, key=lambda fp: fp[0])])
            want = full.tensors[out_role].reshape(-1)
            ok = got.shape == want.shape and torch.equal(got.view(torch.int32), want.view(torch.int32))
            with open(out_path, "w") as f:
                f.write("ok" if ok else f"mismatch: {got.shape} vs {want.shape}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("name,leading,inner", [("rmsnorm", 64, 4096), ("bmm4x4", 1000, 16), ("inv4x4", 1000, 16), ("add", 4096, 1)])
def test_sharded_ranks_reproduce_the_unsharded_result(tmp_path, world, name, leading, inner):
    out = tmp_path / "result.txt"
    mp.spawn(_rank_main, args=(world, _free_port(), name, leading, inner, str(out)), nprocs=world, join=True)
    assert out.read_text() == "ok"
