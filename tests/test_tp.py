"""Tensor-parallel path: host-side sharding logic on CPU (gloo, world size 2) and,
when the box has two GPUs, the real NCCL runner against the oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, rel_l2


def _cpu_rank(rank, world, port, out_q):
    """One CPU rank: its row- and column-shards of a Q4_0 weight through the oracle, combined over gloo."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import tl_ref as ref
    from tensorlogic_b200 import synth
    from tensorlogic_b200.comm import shard_ranges
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, k, m = 64, 1024, 3
    tid = synth.tensor_id("blk.0.ffn_down.weight")
    full = synth.blocks(2, 4, tid, n, k)                   # [n, k/32, 18]
    x = synth.activations(4, "x", (m, k))
    # column-parallel (rows of W): each rank generates ONLY its rows
    r0, r1 = shard_ranges(n, world)[rank]
    mine = synth.blocks(2, 4, tid, n, k, row0=r0, rows=r1 - r0)
    assert np.array_equal(mine, full[r0:r1])
    y_rows = ref.linear_q(2, mine, r1 - r0, k, x)
    gathered = [torch.zeros(m, r1 - r0, dtype=torch.float16) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(y_rows))
    y_col_parallel = torch.cat(gathered, dim=1).numpy()
    # row-parallel (block columns of W): partial products, summed by the all-reduce
    b0, b1 = shard_ranges(k // 32, world)[rank]
    part = ref.linear_q(2, np.ascontiguousarray(full[:, b0:b1]), n, (b1 - b0) * 32, np.ascontiguousarray(x[:, b0 * 32:b1 * 32]))
    acc = torch.from_numpy(part.astype(np.float32))
    dist.all_reduce(acc)
    y_row_parallel = acc.numpy().astype(np.float16)
    if rank == 0:
        want = ref.linear_q(2, full, n, k, x)
        out_q.put((rel_l2(y_col_parallel, want), rel_l2(y_row_parallel, want)))
    dist.barrier()
    dist.destroy_process_group()


def test_sharding_logic_two_cpu_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_cpu_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    e_col, e_row = q.get(timeout=5)
    assert e_col == 0.0          # whole rows: bit-identical to the unsharded product
    assert e_row < 2e-3          # split K: different summation order and one extra f16 rounding per rank


def test_shard_ranges_and_split_rules():
    from tensorlogic_b200 import _lib
    from tensorlogic_b200.comm import combine_row_parallel, shard_ranges
    from tensorlogic_b200.model import LLAMA2_70B, split_for
    assert shard_ranges(8, 4) == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        shard_ranges(10, 4)
    assert split_for("blk.3.attn_q.weight") == _lib.SPLIT_ROWS and split_for("output.weight") == _lib.SPLIT_ROWS
    assert split_for("blk.3.attn_output.weight") == _lib.SPLIT_COLS and split_for("blk.0.ffn_down.weight") == _lib.SPLIT_COLS
    assert split_for("token_embd.weight") == _lib.SPLIT_NONE and split_for("blk.1.attn_norm.weight") == _lib.SPLIT_NONE
    # 70B shapes divide at TP 2/4/8 with whole blocks per rank
    a = LLAMA2_70B
    for tp in (2, 4, 8):
        assert a.n_heads % tp == 0 and a.n_kv_heads % tp == 0 and a.ffn_dim % (32 * tp) == 0 and a.vocab % tp == 0
    parts = [np.full((2, 3), 0.1, np.float16), np.full((2, 3), 0.2, np.float16)]
    assert np.allclose(combine_row_parallel(parts).astype(np.float32), 0.3, atol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_runner_against_oracle(world):
    """tests/tp_parity.py under torchrun at every world size the box has GPUs for: the fused
    all-reduce against a host sum, then prefill + decode logits against the oracle's unsharded
    forward.  At 8 ranks every rank holds one query/KV head and two Q4_0 blocks of attn_output."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                        "--master-addr", "127.0.0.1", "--master-port", str(29517 + world),
                        os.path.join(ROOT, "tests", "tp_parity.py")],
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
