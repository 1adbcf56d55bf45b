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
