"""Distributed vocabulary on the host: planner / topology / analysis logic in-process, tensor
parallelism, the Analyze -> Plan -> Apply flow and pipeline parallelism with gloo ranks."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

from spikingjelly_b200.activation_based import distributed as D
from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
from spikingjelly_b200.parallel import pipeline as PP
from spikingjelly_b200.parallel import tensor_parallel as TP


# ------------------------------------------------------------------------------ in-process logic
def test_topology_and_plan_properties():
    t = D.SNNDistributedTopology.from_mapping({"tp": 2, "dp": 4})
    assert t.world_size == 8 and t.ordered_dim_names == ("dp", "tp") and t.mesh_shape == (4, 2)
    with pytest.raises(ValueError, match="multiply to 6"):
        D.SNNDistributedTopology(world_size=8, dims={"dp": 3, "tp": 2})
    with pytest.raises(TypeError):
        D.SNNDistributedTopology.from_mapping({"dp": True})
    with pytest.raises(ValueError):
        D.SNNDistributedConfig(mode="zz")


def test_recommendations():
    r = D.recommend_snn_distributed_strategy
    assert r("spikformer_ti", 1, "speed", 32).mode == "none"
    s = r("spikformer_ti", 8, "speed", 32)
    assert (s.mode, s.optimizer_sharding, s.dp_mesh_dim) == ("dp", "zero", 0)
    v = r("cifar10dvs_vgg", 4, "speed", 32)
    assert (v.mode, v.mesh_shape, v.tp_mesh_dim, v.dp_mesh_dim) == ("fsdp2_tp", (2, 2), 1, 0)
    m = r("x", 2, "memory", 32)
    assert (m.mode, m.memopt_level, m.mesh_shape) == ("tp", 1, (2,))
    c = r("x", 4, "capacity", 64)
    assert (c.mode, c.pp_virtual_stages, c.pp_schedule, c.pp_microbatches) == ("pp", 2, "interleaved", 32)
    assert r("x", 4, "capacity", 2).mode == "fsdp2_tp"           # batch too small for a pipeline
    assert r("x", 4, "capacity", 64, pipelining_available=False, fsdp2_available=False, tensor_parallel_available=False).mode == "dp"
    with pytest.raises(ValueError):
        r("x", 2, "fast", 8)
    assert D.recommended_pipeline_microbatches(48, 4) == 16
    with pytest.raises(ValueError):
        D.recommended_pipeline_microbatches(3, 4)


def _mlp():
    return nn.Sequential(layer.Linear(16, 32), neuron.LIFNode(surrogate_function=surrogate.ATan()), layer.Dropout(0.0),
                         layer.Linear(32, 32), neuron.LIFNode(surrogate_function=surrogate.ATan()), layer.Linear(32, 8))


def test_analysis_and_planning_rules():
    net = nn.Sequential(layer.Conv2d(1, 2, 3), _mlp())
    a = D.analyze(net)
    assert a.tensor_parallel_candidate_names == ("1.0", "1.3", "1.5") and a.unsupported_tensor_parallel_names == ("0",)
    assert a.memory_module_names == ("1.1", "1.2", "1.4") or "1.1" in a.memory_module_names
    with pytest.raises(KeyError):
        D.analyze(net, roots=["nope"])
    p = D.plan(analysis=a, objective="speed", topology={"dp": 2}, backend="cuda", batch_size=8)
    assert p.mode == "dp" and p.optimizer_strategy == "zero" and p.dp_mesh_dim == 0 and p.tp_mesh_dim == 0
    p = D.plan(analysis=a, objective="speed", topology={"dp": 2}, backend="cuda", batch_size=8, features=D.DistributedFeatureSet(allow_zero_optimizer=False))
    assert p.optimizer_strategy == "none" and any("ZeRO optimizer sharding was switched off" in n for n in p.notes)
    p = D.plan(analysis=a, objective="memory", topology={"tp": 4}, backend="cuda", batch_size=8)
    assert p.mode == "tp" and any("reduced to 'tp'" in n for n in p.notes)
    with pytest.raises(ValueError, match="requires both 'dp' and 'tp'"):
        D.plan(analysis=a, objective="memory", topology={"tp": 4}, backend="cuda", batch_size=8, mode="fsdp2_tp")
    with pytest.raises(NotImplementedError):
        D.plan(analysis=a, objective="memory", topology={"tp": 4}, backend="cuda", batch_size=8, mode="pp")
    with pytest.raises(ValueError, match="outside the analysis candidates"):
        D.plan(analysis=a, objective="memory", topology={"tp": 2}, backend="cuda", batch_size=8, mode="tp", tensor_parallel_plan={"zz": "colwise"})
    empty = D.analyze(nn.Sequential(neuron.IFNode()))
    with pytest.raises(ValueError, match="requires at least one tensor-parallel candidate"):
        D.plan(analysis=empty, objective="memory", topology={"tp": 2}, backend="cuda", batch_size=8, mode="tp")
    assert TP.auto_build_tensor_parallel_plan(_mlp()) == {"0": "colwise_local_output", "3": "colwise_local_output", "5": "rowwise"}


def test_pipeline_partition_helpers():
    assert PP._partition_costs_contiguously([5, 1, 1, 1, 5, 1], 3) == [1, 3, 2]
    assert sum(PP._partition_costs_contiguously([1.0] * 10, 4)) == 10 and PP._partition_costs_contiguously([1, 2], 4) == [1, 1, 0, 0]
    assert PP.parse_pipeline_layout("3|4, 1", 3, 8) == (3, 4, 1)
    with pytest.raises(ValueError):
        PP.parse_pipeline_layout([1, 2], 3, 3)
    assert PP.resolve_pipeline_schedule_kind("auto", 2, False) == "interleaved" and PP.resolve_pipeline_schedule_kind("auto", 2, True) == "zero_bubble"
    with pytest.raises(ValueError):
        PP.resolve_pipeline_schedule_kind("1f1b", 2, False)
    assert D.recommend_pipeline_memopt_stages([1.0, 5.0, 3.0, 2.0], 0.5) == (1, 2)
    with pytest.raises(ValueError):
        D.recommend_pipeline_memopt_stages([1.0], 1.5)


def test_shard_validator_on_one_rank():
    sn = neuron.LIFNode(step_mode="m")
    sharded = D.make_tensor_shard_memory_module(sn, shard_dim=-1, logical_dim_size=32)
    assert sharded is not sn and D.make_tensor_shard_memory_module(sharded, -1, 32) is sharded
    sharded(torch.rand(2, 3, 32))
    with pytest.raises(ValueError, match="Expected local shard size 32"):
        sharded(torch.rand(2, 3, 16))


# ------------------------------------------------------------------------------ multi-process parts
def _init(rank, world, init_file):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)


def _reference_grads(make, x, y):
    torch.manual_seed(0)
    net = make()
    out = net(x)
    ((out.mean(0) - y) ** 2).mean().backward()
    return net, out.detach()


def _tp_worker(rank, world, init_file, out_dir):
    _init(rank, world, init_file)
    torch.manual_seed(7)
    x, y = torch.rand(4, 6, 16), torch.rand(6, 8)

    def make():
        net = _mlp()
        functional.set_step_mode(net, "m")
        return net

    ref, ref_out = _reference_grads(make, x, y)
    torch.manual_seed(0)
    net = make()
    analysis = D.analyze(net)
    plan = D.plan(analysis=analysis, objective="memory", topology={"tp": world}, backend="cpu", batch_size=6, mode="tp")
    D.enable_tp_communication_debug(True)
    D.reset_tp_communication_debug_stats()
    rt = D.apply(model=net, plan=plan, device_type="cpu")
    assert isinstance(rt.model[0], TP.ColwiseParallelLinear) and isinstance(rt.model[5], TP.RowwiseParallelLinear)
    assert rt.model[0].weight.shape == (32 // world, 16) and rt.model[3].weight.shape == (32 // world, 32)
    assert TP._has_validator(rt.model[1])
    out = rt.model(x)
    ((out.mean(0) - y) ** 2).mean().backward()
    stats = D.get_tp_communication_debug_stats()
    res = {"out_err": (out.detach() - ref_out).abs().max().item(), "stats": stats}
    # local weight gradients equal the matching slices of the unsharded model's gradients
    n = 32 // world
    res["g0"] = (rt.model[0].weight.grad - ref[0].weight.grad[rank * n:(rank + 1) * n]).abs().max().item()
    res["g3"] = (rt.model[3].weight.grad - ref[3].weight.grad[rank * n:(rank + 1) * n]).abs().max().item()
    res["g5"] = (rt.model[5].weight.grad - ref[5].weight.grad[:, rank * n:(rank + 1) * n]).abs().max().item()
    opt = rt.build_optimizer(lr=0.01)
    opt.step()
    rt.reset_state()
    logits, target = rt.prepare_classification_output(out.detach(), torch.nn.functional.one_hot(torch.arange(6) % 8, 8))
    res["logits_shape"], res["target"] = tuple(logits.shape), target.tolist()
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_tensor_parallel_mlp_matches_unsharded_model():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_tp_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        for r in range(world):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            assert res["out_err"] < 1e-5 and max(res["g0"], res["g3"], res["g5"]) < 1e-5, res
            assert res["stats"]["all_reduce_calls"] >= 2 and res["stats"]["all_gather_calls"] >= 1
            assert res["logits_shape"] == (6, 8) and res["target"] == [0, 1, 2, 3, 4, 5]


def _conv_spikformer_worker(rank, world, init_file, out_dir):
    _init(rank, world, init_file)
    from spikingjelly_b200.models import spikformer
    res = {}
    # convolution chain
    torch.manual_seed(0)
    def make_conv():
        net = nn.Sequential(layer.Conv2d(2, 8, 3, padding=1, bias=False), layer.BatchNorm2d(8), neuron.IFNode(), layer.MaxPool2d(2),
                            layer.Conv2d(8, 4, 3, padding=1), layer.BatchNorm2d(4), neuron.IFNode())
        functional.set_step_mode(net, "m")
        return net
    torch.manual_seed(1)
    x = torch.rand(3, 2, 2, 8, 8)
    torch.manual_seed(0); ref = make_conv(); ref_out = ref(x); ref_out.sum().backward()
    torch.manual_seed(0); net = make_conv()
    net = TP.parallelize_snn_conv_blocks(nn.Sequential(net), None, roots=["0"])[0]
    assert isinstance(net[0], TP.ChannelShardConv2d) and net[0].weight.shape[0] == 8 // world and isinstance(net[4], TP.ChannelShardConv2d)
    out = net(x); out.sum().backward()
    res["conv_err"] = (out - ref_out).abs().max().item()
    res["conv_g"] = (net[4].weight.grad - ref[4].weight.grad[:, rank * 4:(rank + 1) * 4]).abs().max().item()
    # Spikformer blocks + patch stem
    torch.manual_seed(0)
    kw = dict(img_size_h=32, img_size_w=32, patch_size=16, embed_dims=32, num_heads=4, depths=2, num_classes=5, T=2)
    def make_sf():
        torch.manual_seed(3)
        m = spikformer.Spikformer(**kw)
        m.fused = False
        return m.eval()
    img = torch.rand(2, 3, 32, 32)
    with torch.no_grad():
        ref_logits = make_sf()(img)
        sharded = make_sf()
        TP.parallelize_spikformer_blocks(sharded, None)
        TP.parallelize_spikformer_patch_stem(sharded, None)
        res["sf_err"] = (sharded(img) - ref_logits).abs().max().item()
        res["heads"] = sharded.blocks[0].attn.num_heads
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_channel_sharded_convs_and_spikformer_blocks_are_function_preserving():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_conv_spikformer_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        for r in range(world):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            assert res["conv_err"] < 1e-5 and res["conv_g"] < 1e-4 and res["sf_err"] < 1e-4 and res["heads"] == 2, res


def _pp_worker(rank, world, init_file, out_dir):
    _init(rank, world, init_file)
    torch.manual_seed(0)
    units = [nn.Sequential(layer.Linear(8, 16), neuron.LIFNode(surrogate_function=surrogate.ATan())),
             nn.Sequential(layer.Linear(16, 16), neuron.LIFNode(surrogate_function=surrogate.ATan())),
             nn.Sequential(layer.Linear(16, 16), neuron.LIFNode(surrogate_function=surrogate.ATan())),
             layer.Linear(16, 4)]
    full = nn.Sequential(*units)
    x = torch.rand(8, 8)
    y = torch.randint(0, 4, (8,))
    # unsharded reference: mean of the per-micro-batch losses, neurons reset between micro-batches
    ref_loss = 0.0
    for xb, yb in zip(x.chunk(4), y.chunk(4)):
        functional.reset_net(full)
        loss = torch.nn.functional.cross_entropy(full(xb), yb) / 4
        loss.backward()
        ref_loss += float(loss)
    ref_grads = [p.grad.clone() for p in full.parameters()]
    full.zero_grad()
    functional.reset_net(full)
    rt = PP.configure_snn_pipeline(units, x, n_microbatches=4, device="cpu", schedule_kind="gpipe", layout="2|2",
                                   loss_fn=torch.nn.functional.cross_entropy)
    losses = rt.step(x if rt.is_first else None, y if rt.is_last else None)
    res = {"stage": rt.local_stage_indices, "num_stages": rt.num_stages, "first": rt.is_first, "last": rt.is_last}
    if rt.is_last:
        res["loss_err"] = abs(sum(float(l) for l in losses) / 4 - ref_loss)
    mine = [p.grad for s in rt.stage_modules for p in s.parameters()]
    ref_slice = ref_grads[:4] if rank == 0 else ref_grads[4:]
    res["grad_err"] = max((a / 1.0 - b).abs().max().item() for a, b in zip(mine, ref_slice))
    res["memopt"] = D.recommend_pipeline_memopt_stages(rt.stage_costs or (1.0, 2.0), 0.5)
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_pipeline_parallel_matches_microbatched_reference():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_pp_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        r0, r1 = (torch.load(os.path.join(d, f"r{r}.pt")) for r in range(world))
    assert r0["first"] and not r0["last"] and r1["last"] and r0["num_stages"] == 2
    assert r1["loss_err"] < 1e-5
    assert r0["grad_err"] < 1e-4 and r1["grad_err"] < 1e-4, (r0, r1)
