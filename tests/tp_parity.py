"""Tensor-parallel parity check, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/tp_parity.py

Every rank builds its shard of a small LLaMA (weights split Megatron-style), joins
the communicator (NCCL + the peer-memory exchange), checks the fused all-reduce +
residual kernel against a host sum, runs prefill + greedy decode, and compares its
logits with the CPU oracle's unsharded forward (rank 0 prints PASS/FAIL; exit code says the same).
The id of the communicator travels over torch.distributed's gloo backend.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def main() -> int:
    import torch.distributed as dist
    import tl_ref as ref
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import Device
    from tensorlogic_b200.comm import Comm, unique_id
    from tensorlogic_b200.model import Llama, LlamaArch, model_from_host, synthetic_host_weights

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")
    dev = Device(local)
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Comm(dev, box[0], rank, world)

    def gather(blob):
        out = [None] * world
        dist.all_gather_object(out, blob)
        return out

    # residual + all-reduce before and after the peer-memory exchange exists (NCCL + add, then one kernel)
    rng = np.random.default_rng(100 + rank)
    failed = []                                               # names of the checks this rank failed

    def check(name, cond):
        if not bool(cond):
            failed.append(name)

    # nccl: library all-reduce + add; p2p: flagged words over peer memory (no fences);
    # p2p-fenced: the store + fence + flag form longer vectors use; p2p-too-large: back to NCCL
    for phase in ("nccl", "p2p", "p2p-fenced", "p2p-too-large"):
        if phase == "p2p":
            comm.enable_p2p(65536, gather)
            check("p2p_ready", comm.p2p_ready)
        dev.set_option("comm_ll", 0 if phase == "p2p-fenced" else 1)
        for rep, n in enumerate((8, 40, 1024, 4096, 4096, 2048, 65536, 2048, 65536, 8) if phase != "p2p-too-large" else (131072,)):
            part = rng.standard_normal(n).astype(np.float16)
            res = np.random.default_rng(7 * rep + n).standard_normal(n).astype(np.float16)  # same on every rank
            parts = gather(part.tobytes())
            acc = np.zeros(n, np.float32)
            for b in parts:                                   # rank order, f32, one rounding
                acc += np.frombuffer(b, np.float16).astype(np.float32)
            want_sum = acc.astype(np.float16)
            got = comm.all_reduce_residual(dev.tensor(part), dev.tensor(res)).numpy()
            got_sum = comm.all_reduce_residual(dev.tensor(part)).numpy()
            if phase == "nccl" or phase == "p2p-too-large":   # the library's own f16 summation order
                # f16 partial sums inside the library: a few f16 roundings of values up to ~world * 3
                check(f"{phase} sum n={n}", np.allclose(got_sum.astype(np.float32), acc, rtol=1e-2, atol=8e-3 * world))
                check(f"{phase} sum+residual n={n}",
                      np.allclose(got.astype(np.float32), acc + res.astype(np.float32), rtol=1e-2, atol=8e-3 * world))
            else:
                check(f"{phase} sum n={n} rep={rep} (bit-exact)", np.array_equal(got_sum.view(np.uint16), want_sum.view(np.uint16)))
                check(f"{phase} sum+residual n={n} rep={rep} (bit-exact)",
                      np.array_equal(got.view(np.uint16), (res + want_sum).view(np.uint16)))
    dev.synchronize()

    # all-reduce / all-gather on their own
    t = dev.tensor(np.full((3, 5), rank + 1, np.float16))
    comm.all_reduce(t)
    check("all_reduce", np.all(t.numpy() == np.float16(world * (world + 1) / 2)))
    g = comm.all_gather(dev.tensor(np.full((4,), rank, np.float16))).numpy()
    check("all_gather", np.array_equal(g, np.repeat(np.arange(world, dtype=np.float16), 4).reshape(world, 4)))

    arch = LlamaArch(n_layers=3, d_model=512, n_heads=8, n_kv_heads=8 if world > 4 else 4, head_dim=64,
                     ffn_dim=1024, vocab=2048)
    weights = synthetic_host_weights(arch, seed=9)
    model = model_from_host(dev, weights, tp_rank=rank, tp_size=world)
    llm = Llama(dev, model, arch, max_seq=96, max_prefill=32, logits_all_rows=True, tp_rank=rank, tp_size=world)
    llm.set_comm(comm)
    ids = synth.token_ids(9, "prompt", 21, arch.vocab)
    nxt, logits = llm.prefill(ids, all_rows=True)

    errs = []
    if rank == 0:
        rw = {n: (a.reshape(-1) if n.endswith("norm.weight") else a) if t_ == 1 else (t_, a, (a.shape[0], a.shape[1] * 32))
              for n, (t_, a) in weights.items()}
        oracle = ref.RefLlama(rw, arch.n_layers, arch.n_heads, arch.n_kv_heads, arch.head_dim, arch.rms_eps, arch.rope_base)
        want = oracle.forward(ids)
        rel = lambda a, b: float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) /
                                 np.linalg.norm(b.astype(np.float64)))
        errs.append(rel(logits, want))
        check("prefill token == argmax of own logits", nxt == ref.argmax_last(logits[-1]))
        tok = ref.argmax_last(want[-1])
    else:
        tok = 0
    box = [tok]
    for step in range(4):
        dist.broadcast_object_list(box, src=0)       # teacher-forced with the oracle's token
        got, lg = llm.decode([box[0]], return_logits=True)
        if rank == 0:
            w = oracle.forward([box[0]])
            errs.append(rel(lg, w))
            check(f"decode step {step}: token == argmax of own logits", int(got[0]) == ref.argmax_last(lg[0]))
            box = [ref.argmax_last(w[0])]
    # every rank must hold the same full logits and the same sampled token
    all_lg = [None] * world
    dist.all_gather_object(all_lg, (lg.tobytes(), int(got[0])))
    check("same logits and token on every rank", all(a == all_lg[0] for a in all_lg))
    flags = [None] * world
    dist.all_gather_object(flags, list(failed))
    ok = not any(flags)
    if rank == 0:
        for r, f in enumerate(flags):
            if f:
                print(f"rank {r} failed: {f}", flush=True)
        ok = ok and max(errs) < 1e-2
        print(f"tp={world} rel-L2 of logits vs oracle: {['%.2e' % e for e in errs]}  {'PASS' if ok else 'FAIL'}",
              flush=True)
    flag = [bool(ok)]
    dist.broadcast_object_list(flag, src=0)
    dev.synchronize()
    dist.destroy_process_group()
    return 0 if flag[0] else 1


if __name__ == "__main__":
    sys.exit(main())
