"""SNNDataParallel bucket/hook logic with real processes on the gloo backend (CPU).
The fused NVLink kernel is replaced by dist.all_reduce there; everything else is identical."""
import os
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _worker(rank, world, init_file, out_dir):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
    from spikingjelly_b200.parallel.data_parallel import SNNDataParallel
    torch.manual_seed(100 + rank)                      # different init per rank: broadcast must fix it
    net = nn.Sequential(layer.Linear(12, 16), neuron.LIFNode(surrogate_function=surrogate.ATan()),
                        layer.Linear(16, 4), neuron.LIFNode(surrogate_function=surrogate.ATan()))
    functional.set_step_mode(net, "m")
    dp = SNNDataParallel(net, bucket_cap_mb=0.0005)    # tiny cap -> several buckets
    assert len(dp.buckets) >= 2
    opt = torch.optim.SGD(dp.parameters(), lr=0.1)
    torch.manual_seed(7)
    full_x = torch.rand(3, 4, 8, 12)                   # [step, T, global batch, features]
    full_y = torch.rand(3, 8, 4)
    for step in range(3):
        x = full_x[step][:, rank::world]
        y = full_y[step][rank::world]
        loss = ((dp(x).mean(0) - y) ** 2).mean()
        opt.zero_grad(set_to_none=(step == 1))         # exercise both zero_grad flavours
        loss.backward()
        opt.step()
        functional.reset_net(net)
    torch.save({k: v.clone() for k, v in net.state_dict().items()}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def _single_process_reference():
    from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
    torch.manual_seed(100)                             # rank 0's initial weights
    net = nn.Sequential(layer.Linear(12, 16), neuron.LIFNode(surrogate_function=surrogate.ATan()),
                        layer.Linear(16, 4), neuron.LIFNode(surrogate_function=surrogate.ATan()))
    functional.set_step_mode(net, "m")
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    torch.manual_seed(7)
    full_x = torch.rand(3, 4, 8, 12)
    full_y = torch.rand(3, 8, 4)
    for step in range(3):
        loss = ((net(full_x[step]).mean(0) - full_y[step]) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        functional.reset_net(net)
    return net.state_dict()


def test_two_ranks_match_single_process():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "init")
        mp.spawn(_worker, args=(world, init_file, d), nprocs=world, join=True)
        sds = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(world)]
    ref = _single_process_reference()
    for k in ref:
        assert torch.equal(sds[0][k], sds[1][k]), k                 # ranks stay in lock step
        torch.testing.assert_close(sds[0][k], ref[k], rtol=1e-5, atol=1e-6)   # mean of shard grads == full-batch grad


def test_epoch_counter_wraps_like_the_device_compare():
    """The device predicate is ``(int32)(flag - epoch) >= 0`` on uint32 values; the host counter must wrap
    modulo 2^32 for it to stay correct across the wrap."""
    from spikingjelly_b200.parallel.comm import EPOCH_MASK, epoch_reached, next_epoch
    assert EPOCH_MASK == 0xFFFFFFFF
    e = 0xFFFFFFFD                                     # phase 2 of this call uses e + 1
    nxt = next_epoch(e, 2)
    assert nxt == 0xFFFFFFFF and next_epoch(nxt, 2) == 1
    # a slot that still holds the previous call's phase-2 value has NOT reached the next epoch ...
    last_phase2 = (nxt + 1) & EPOCH_MASK               # 0 after the wrap
    assert last_phase2 == 0 and not epoch_reached(last_phase2, next_epoch(nxt, 2))
    # ... a peer that is one collective ahead has, and a 31-bit wrap would have got this wrong
    assert epoch_reached(3, 1) and epoch_reached(1, 1) and not epoch_reached(0xFFFFFFFF, 1)
    assert not epoch_reached(0x80000000, 1 + 0x7FFFFFFF + 2)


def test_bucket_plan_keeps_the_last_bucket_small():
    from spikingjelly_b200.parallel.data_parallel import plan_buckets
    sizes = [100, 50, 4000, 4000, 4000, 300]           # registration order; index 0's gradient arrives last
    plan = plan_buckets(sizes, cap=8000, tail_cap=200)
    assert sorted(i for g in plan for i in g) == list(range(6))
    assert plan[-1] == [1, 0]                          # 150 elements, exchanged last
    assert plan[0][0] == 5                             # reverse registration order first
    assert all(sum(sizes[i] for i in g) <= 8000 for g in plan)
    # nothing fits under the tail cap: the plan is the plain reverse-order grouping
    assert plan_buckets([500, 500], cap=600, tail_cap=10) == [[1], [0]]
    assert plan_buckets([7], cap=1, tail_cap=100) == [[0]]


def _failed_exchange_worker(rank, world, init_file, out_dir):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    from spikingjelly_b200.parallel.comm import CommError
    from spikingjelly_b200.parallel.data_parallel import SNNDataParallel
    torch.manual_seed(0)
    net = nn.Linear(4, 3)
    dp = SNNDataParallel(net, timeout_s=1.0)
    opt = torch.optim.SGD(dp.parameters(), lr=1.0)
    dp.guard_optimizer(opt, strict=True)
    dp(torch.ones(2, 4)).sum().backward()
    before = net.weight.detach().clone()
    # what the kernel leaves behind when its wait on rank 1 runs out (phase 1, block 0)
    dp.status.dev.copy_(torch.tensor([1, rank, 1 - rank, 0], dtype=torch.int32))
    dp.status.mirror()
    outcome = {}
    try:
        opt.step()
        outcome["step"] = "stepped"
    except CommError as e:
        outcome["step"] = f"CommError: {e}"
    outcome["weights_unchanged"] = bool(torch.equal(before, net.weight.detach()))
    # the record is consumed: the next step runs normally
    dp(torch.ones(2, 4)).sum().backward()
    opt.step()
    outcome["recovered"] = not torch.equal(before, net.weight.detach())
    # the same record is also seen at the start of forward
    dp.status.dev.copy_(torch.tensor([2, rank, 1 - rank, 3], dtype=torch.int32))
    dp.status.mirror()
    try:
        dp(torch.ones(2, 4))
        outcome["forward"] = "ran"
    except CommError as e:
        outcome["forward"] = f"CommError: {e}"
    torch.save(outcome, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_failed_exchange_raises_instead_of_stepping_the_optimizer():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_failed_exchange_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        outs = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(world)]
    for r, o in enumerate(outs):
        assert o["step"].startswith("CommError") and "bucket" in o["step"], o
        assert o["weights_unchanged"] and o["recovered"], o
        assert o["forward"].startswith("CommError") and "results" in o["forward"], o
