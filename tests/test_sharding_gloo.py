"""The N > 1 path on CPU: two gloo ranks shard a batch, evaluate their shard, gather, and the result
equals the unsharded evaluation.  (On GPUs the per-rank evaluation is the CUDA plan; here the
oracle stands in so that the sharding / gather logic itself is what is under test.)"""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    from aie4ml_b200 import from_graph
    from aie4ml_b200 import workloads as W
    from aie4ml_b200.sharding import gather_outputs, shard_inputs, shard_rows
    from oracle import oracle

    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    total = 37
    _, inputs = W.wide_mlp_cfg5(total)
    s, e = shard_rows(total, rank, world)
    builder, _ = W.wide_mlp_cfg5(e - s)          # same seed -> same weights on every rank
    plan = from_graph(builder).export_plan()
    local = oracle.run_plan(plan, shard_inputs(inputs, rank, world))
    (name, y), = local.items()
    full = gather_outputs(torch.from_numpy(np.ascontiguousarray(y)), total)
    np.save(Path(out_dir) / f'rank{rank}.npy', full.numpy())
    # equal shards gather straight into the result (no padding, no trim), also from a strided view
    even = 2 * (total // 2)
    s2, e2 = shard_rows(even, rank, world)
    wide = torch.arange(even * 16, dtype=torch.int32).reshape(even, 16)
    part = wide[s2:e2, :10]                       # a row pitch wider than the rows, like a 10-wide output in a 16-byte pitch
    np.save(Path(out_dir) / f'even{rank}.npy', gather_outputs(part, even).numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_and_gather_equals_unsharded(tmp_path):
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    sys.path.insert(0, str(ROOT))
    from aie4ml_b200 import from_graph
    from aie4ml_b200 import workloads as W
    from oracle import oracle

    builder, inputs = W.wide_mlp_cfg5(37)
    want = next(iter(oracle.run_plan(from_graph(builder).export_plan(), inputs).values()))
    for r in range(2):
        np.testing.assert_array_equal(np.load(tmp_path / f'rank{r}.npy'), want)
        np.testing.assert_array_equal(np.load(tmp_path / f'even{r}.npy'), np.arange(36 * 16, dtype=np.int32).reshape(36, 16)[:, :10])
