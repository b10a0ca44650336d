"""One rank of the data-parallel parity check, launched by torchrun (see test_gpu_data_parallel).

Every rank trains the BERT twin on its shard of a global batch through the C ABI, gradients
bucket-all-reduced over NCCL; rank 0 also runs the CPU oracle on the whole batch as one device
would see it, and compares losses and parameters within the run tolerance. torch.distributed is
only the plumbing that carries the communicator id and the barrier."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    import torch
    import torch.distributed as dist
    import modelspec_b200 as M
    from modelspec_b200 import models, synthetic

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    steps, batch, seq, vocab = 12, 4, 16, 300
    kw = dict(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=vocab, seq=seq, lr=3e-3, warmup_steps=2, steps=steps)
    local_source = models.bert(batch=batch, **kw)
    rows = batch * seq
    capacity = 32
    device = M.Device(local)
    run = M.Training(device, local_source, capacity)
    ids = [M.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    run.comm_init(rank, world, ids[0], rows)
    feed = lambda k: synthetic.mlm_batch(k, vocab=vocab, seq=seq, batch=batch * world)
    shard = lambda full: {name: value[rank * rows:(rank + 1) * rows] for name, value in full.items()}
    losses = []
    for k in range(steps):
        for name, value in shard(feed(k)).items():
            run.set_input(name, value)
        run.step(k, steps)
        losses.append(float(run.loss()))
    for name, value in shard(feed(steps)).items():
        run.set_input(name, value)
    losses.append(float(run.final_loss()))
    params = [run.step_plan.param_download(i) for i in range(len(run.step_plan.params()))]
    buckets = M.lib().msx_comm_bucket_count(run.step_plan.h)
    # Every rank holds the same parameters after every step.
    for p in params:
        t = torch.from_numpy(p.copy())
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "ranks disagree on a parameter"
    ok = True
    if rank == 0:
        import oracle_lib
        from helpers import assert_run_close
        cpu = oracle_lib.Trainer(models.bert(batch=batch * world, **kw), capacity * world)
        cpu_losses = []
        for k in range(steps):
            for name, value in feed(k).items():
                cpu.set_input(name, value)
            cpu_losses.append(float(cpu.step(k, steps)))
        for name, value in feed(steps).items():
            cpu.set_input(name, value)
        cpu_losses.append(float(cpu.final_loss()))
        try:
            assert_run_close(np.array(losses), np.array(cpu_losses), "data-parallel losses")
            for i, path in enumerate(cpu.param_paths()):
                atol = 1e-4 + steps * 3e-3 * 1e-3 if path.endswith("_bk") else 1e-4
                assert_run_close(params[i], cpu.read("param", i), "data-parallel parameter " + path, atol=atol)
            exchange = "peer" if M.lib().msx_comm_uses_peer_memory(run.step_plan.h) else "nccl"
            print("DP_PARITY_OK world=%d buckets=%d exchange=%s last_loss=%.6f cpu=%.6f" % (world, buckets, exchange, losses[-1], cpu_losses[-1]), flush=True)
        except AssertionError as e:
            ok = False
            print("DP_PARITY_FAILED", e, flush=True)
    run.destroy()
    device.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
