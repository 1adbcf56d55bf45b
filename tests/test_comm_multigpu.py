"""The fused NVLink all-reduce kernel and SNNDataParallel on 2+ real GPUs (one process per GPU).

The failure case is produced on the host: one rank simply does not join a collective (its process
stays alive and idle), the other rank's bounded device wait expires and reports a status code.
No GPU is made to fault; NVLS is off and the kernel uses plain peer loads in that test.
"""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _init(rank, world, init_file):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))


def _allreduce_worker(rank, world, init_file, out_dir, use_multimem, wire):
    _init(rank, world, init_file)
    from spikingjelly_b200.parallel.comm import SymmetricBucket
    dev = torch.device("cuda", rank)
    results = {}
    for numel in (4, 1000, 1 << 20, (1 << 22) + 12):
        bucket = SymmetricBucket(numel, dev, use_multimem=use_multimem, wire=wire, timeout_s=20.0)
        results[f"multimem_{numel}"] = bucket.uses_multimem
        for it in range(3):                                      # repeated calls advance the flag epoch
            g = torch.Generator(device="cpu").manual_seed(1000 * it + numel)
            contributions = [torch.randn(bucket.numel, generator=g) for _ in range(world)]
            bucket.buffer.copy_(contributions[rank])
            bucket.all_reduce_(1.0 / world)
            bucket.check()
            if wire == "bf16":                                   # summands and the mean are rounded to bf16 on the wire
                contributions = [c.bfloat16().float() for c in contributions]
            expect = torch.stack(contributions).sum(0) / world
            if wire == "bf16":
                expect = expect.bfloat16().float()
            err = (bucket.buffer.cpu() - expect).abs().max().item()
            results[f"err_{numel}_{it}"] = err
            dist.barrier()                                       # nobody refills its bucket while a peer still reads it
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("wire", ["fp32", "bf16"])
@pytest.mark.parametrize("use_multimem", [False, True])
def test_fused_allreduce_matches_sum(use_multimem, wire):
    world = min(torch.cuda.device_count(), 4)
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_allreduce_worker, args=(world, os.path.join(d, "init"), d, use_multimem, wire), nprocs=world, join=True)
        for r in range(world):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            errs = {k: v for k, v in res.items() if k.startswith("err_")}
            # bf16 wire: the in-switch sum may round differently from the host's fp32 sum by one bf16 ulp of ~4
            assert errs and max(errs.values()) < (1e-5 if wire == "fp32" else 4e-2), errs


def _dp_worker(rank, world, init_file, out_dir):
    _init(rank, world, init_file)
    from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
    from spikingjelly_b200.parallel.data_parallel import SNNDataParallel
    dev = torch.device("cuda", rank)
    torch.manual_seed(100 + rank)
    net = nn.Sequential(layer.Linear(32, 64), neuron.LIFNode(surrogate_function=surrogate.ATan()),
                        layer.Linear(64, 8), neuron.LIFNode(surrogate_function=surrogate.ATan())).to(dev)
    functional.set_step_mode(net, "m")
    dp = SNNDataParallel(net, bucket_cap_mb=0.005, tail_bucket_mb=0.0005, timeout_s=20.0)
    opt = torch.optim.SGD(dp.parameters(), lr=0.1)
    dp.guard_optimizer(opt, strict=(rank == 0))
    assert len(dp.buckets) >= 2
    torch.manual_seed(7)
    full_x, full_y = torch.rand(3, 4, 8 * world, 32), torch.rand(3, 8 * world, 8)
    for step in range(3):
        x, y = full_x[step][:, rank::world].to(dev), full_y[step][rank::world].to(dev)
        loss = ((dp(x).mean(0) - y) ** 2).mean()
        opt.zero_grad(set_to_none=(step % 2 == 0))               # both ways of clearing gradients
        loss.backward()
        opt.step()
        functional.reset_net(net)
    dp.check_communication()
    torch.save({k: v.cpu() for k, v in net.state_dict().items()}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_matches_single_gpu():
    from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_dp_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        states = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(world)]
    for k in states[0]:
        assert torch.equal(states[0][k], states[1][k]), k        # ranks stay in lock step
    torch.manual_seed(100)
    net = nn.Sequential(layer.Linear(32, 64), neuron.LIFNode(surrogate_function=surrogate.ATan()),
                        layer.Linear(64, 8), neuron.LIFNode(surrogate_function=surrogate.ATan())).cuda()
    functional.set_step_mode(net, "m")
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    torch.manual_seed(7)
    full_x, full_y = torch.rand(3, 4, 8 * world, 32), torch.rand(3, 8 * world, 8)
    for step in range(3):
        loss = ((net(full_x[step].cuda()).mean(0) - full_y[step].cuda()) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        functional.reset_net(net)
    for k, v in net.state_dict().items():
        torch.testing.assert_close(states[0][k], v.cpu(), rtol=1e-4, atol=1e-5)


def _absent_peer_worker(rank, world, init_file, out_dir):
    _init(rank, world, init_file)
    from spikingjelly_b200.parallel.comm import CommError, SymmetricBucket
    dev = torch.device("cuda", rank)
    bucket = SymmetricBucket(4096, dev, use_multimem=False, timeout_s=0.5)
    bucket.buffer.fill_(float(rank + 1))
    bucket.all_reduce_(1.0)                                      # a healthy round first
    bucket.check()
    ok_first = bool((bucket.buffer == 3.0).all())
    dist.barrier()
    outcome = "idle"
    if rank == 0:                                                # rank 1 sits this one out (alive, nothing in flight)
        bucket.all_reduce_(1.0)
        try:
            bucket.check()
            outcome = "no error"
        except CommError as e:
            outcome = f"CommError: {e}"
        # the exchange was skipped: nothing of the absent peer's (unfinished) bucket was summed in
        outcome += f" | untouched={bool((bucket.buffer == 3.0).all())}"
        still_usable = float((torch.ones(8, device=dev) * 2).sum())   # the context survived
        outcome += f" | usable={still_usable}"
    torch.save({"ok_first": ok_first, "outcome": outcome}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_absent_peer_is_reported_not_hung():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_absent_peer_worker, args=(2, os.path.join(d, "init"), d), nprocs=2, join=True)
        r0, r1 = (torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2))
    assert r0["ok_first"] and r1["ok_first"]
    assert r0["outcome"].startswith("CommError") and "rank 1" in r0["outcome"] and "usable=16.0" in r0["outcome"], r0
    assert "untouched=True" in r0["outcome"], r0
    assert r1["outcome"] == "idle"
