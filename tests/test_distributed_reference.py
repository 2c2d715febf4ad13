"""The eager TP x PP reference over gloo equals the single-process eager decoder."""
import datetime
import multiprocessing as mp
import os
import socket

import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec


def _cfg():
    return ModelConfig(name="dist-toy", num_layers=4, hidden_size=64, num_q_heads=4, num_kv_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=128, rope_theta=1e4, qk_norm=True, quant=QuantSpec("none", 16, 0))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, tp, pp, port, q):
    import torch.distributed as dist
    from cubic_serve_b200.models.distributed_reference import DistributedEagerDecoder
    from cubic_serve_b200.models.parallel_weights import plan_partition
    from cubic_serve_b200.models.reference import random_dense_weights
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    torch.set_num_threads(1)
    cfg = _cfg()
    plan = plan_partition(cfg, tp, pp)
    groups = [dist.new_group(list(range(s * tp, (s + 1) * tp))) for s in range(pp)]     # every rank creates every group
    dec = DistributedEagerDecoder(cfg, plan, rank, random_dense_weights(cfg, seed=5, std=0.08), groups[rank // tp])
    prompts = torch.tensor([[3, 17, 99, 4, 56], [8, 8, 120, 33, 2]])
    toks, logits = dec.generate(prompts, 6)
    q.put((rank, toks.tolist(), None if logits[0] is None else torch.stack(logits, 1)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("tp,pp", [(2, 1), (2, 2)])
def test_distributed_reference_equals_single_process(tp, pp):
    from cubic_serve_b200.models.reference import EagerDecoder, random_dense_weights
    cfg = _cfg()
    want_toks, want_logits = EagerDecoder(cfg, random_dense_weights(cfg, seed=5, std=0.08)).generate(
        torch.tensor([[3, 17, 99, 4, 56], [8, 8, 120, 33, 2]]), 6)
    world = tp * pp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, world, tp, pp, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=180) for _ in procs), key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
    for rank, toks, logits in got:
        assert toks == want_toks.tolist(), rank                   # every rank decoded the same tokens
        if rank >= (pp - 1) * tp:                                 # last stage: full-vocabulary logits, rank-order sums
            assert logits is not None and torch.allclose(logits, want_logits, rtol=1e-4, atol=1e-5)
        else:
            assert logits is None
    last = [l for r, _, l in got if r >= (pp - 1) * tp]
    assert all(torch.equal(last[0], l) for l in last[1:])         # identical bits on all tensor ranks


def test_shards_follow_the_ownership_plan():
    from cubic_serve_b200.models.distributed_reference import shard_dense_weights
    from cubic_serve_b200.models.parallel_weights import plan_partition
    from cubic_serve_b200.models.reference import random_dense_weights
    cfg = _cfg()
    w = random_dense_weights(cfg, seed=1)
    plan = plan_partition(cfg, 2, 2)
    s = shard_dense_weights(w, cfg, plan.ranks[3])                # stage 1, tensor rank 1
    assert len(s.layers) == 2
    assert torch.equal(s.layers[0].wq, w.layers[2].wq[32:64]) and torch.equal(s.layers[0].wo, w.layers[2].wo[:, 32:64])
    assert torch.equal(s.layers[1].w_down, w.layers[3].w_down[:, 64:128]) and s.layers[1].wk.shape == (16, 64)


def _moe_rank(rank, world, port, q):
    import torch.distributed as dist
    from cubic_serve_b200.models.distributed_reference import moe_expert_parallel_reference
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(11)
    E, H, I, T = 8, 32, 48, 9
    router = (torch.randn(E, H, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = [(torch.randn(2 * I, H, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    down = [(torch.randn(H, I, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    per = E // world
    y = moe_expert_parallel_reference(x, router, gate_up[rank * per:(rank + 1) * per], down[rank * per:(rank + 1) * per],
                                      2, dist.group.WORLD)
    q.put((rank, y))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_reference_equals_the_single_process_block():
    from cubic_serve_b200.models.moe import moe_reference
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_moe_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    g = torch.Generator().manual_seed(11)
    E, H, I, T = 8, 32, 48, 9
    router = (torch.randn(E, H, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = [(torch.randn(2 * I, H, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    down = [(torch.randn(H, I, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    want = moe_reference(x, router, gate_up, down, 2)
    assert torch.equal(got[0], got[1])                      # rank-ordered sum: the same bits on every rank
    assert float((got[0] - want).norm() / want.norm()) < 1e-5


def _moe_etp_rank(rank, world, port, q):
    import torch.distributed as dist
    from cubic_serve_b200.models.distributed_reference import moe_expert_parallel_reference
    from cubic_serve_b200.models.moe import expert_coordinates
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(13)
    E, H, I, T = 8, 32, 48, 9
    router = (torch.randn(E, H, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = [(torch.randn(2 * I, H, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    down = [(torch.randn(H, I, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    owner, lane, lanes = expert_coordinates(rank, world, 2)          # 2 owners x 2 lanes
    per, il = E // 2, I // lanes
    mine = range(owner * per, (owner + 1) * per)
    gu = [torch.cat([gate_up[e][lane * il:(lane + 1) * il], gate_up[e][I + lane * il:I + (lane + 1) * il]]) for e in mine]
    dn = [down[e][:, lane * il:(lane + 1) * il] for e in mine]
    y = moe_expert_parallel_reference(x, router, gu, dn, 2, dist.group.WORLD, ep_size=2)
    q.put((rank, y))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_tensor_lanes_complete_the_experts():
    """Two expert owners times two lanes: every lane holds half of each owned expert's features; the sum over the four
    ranks is the whole block (each lane rounds its partial expert output to bf16, hence the tolerance)."""
    from cubic_serve_b200.contracts.execution import ParallelTopology
    from cubic_serve_b200.models.moe import expert_coordinates, moe_reference
    world = 4
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_moe_etp_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    g = torch.Generator().manual_seed(13)
    E, H, I, T = 8, 32, 48, 9
    router = (torch.randn(E, H, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = [(torch.randn(2 * I, H, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    down = [(torch.randn(H, I, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    want = moe_reference(x, router, gate_up, down, 2)
    assert all(torch.equal(got[0], got[r]) for r in range(1, world))
    assert float((got[0] - want).norm() / want.norm()) < 5e-3
    topo = ParallelTopology.single_node(range(4), tp=4, ep=2)
    for r in range(4):
        owner, lane, lanes = expert_coordinates(r, 4, 2)
        assert (topo.placement(r).expert_rank, topo.placement(r).expert_tensor_rank, topo.etp) == (owner, lane, lanes)
        assert topo.expert_slice(r, 8) == (owner * 4, owner * 4 + 4)
        assert topo.expert_feature_slice(r, 48) == (lane * 24, lane * 24 + 24)
    with pytest.raises(ValueError):
        expert_coordinates(0, 4, 3)


def test_random_expert_shards_with_lanes_are_slices_of_one_model():
    from dataclasses import replace

    from cubic_serve_b200.models.config import ModelConfig, QuantSpec
    from cubic_serve_b200.models.moe import moe_reference, random_moe_weights
    from cubic_serve_b200.ops import wq_pack
    cfg = replace(ModelConfig(), family="gqa_moe", hidden_size=128, num_experts=4, experts_per_token=2,
                  moe_intermediate_size=256, quant=QuantSpec("none", 16, 0))
    gen = torch.Generator()
    x = (torch.randn(6, 128, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)

    def dense(layer):
        gu = wq_pack.unpack_to_dense(layer.gate_up)
        dn = wq_pack.unpack_to_dense(layer.down)
        return (layer.router, list(gu.view(layer.expert_count, -1, gu.shape[-1])),
                list(dn.view(layer.expert_count, -1, dn.shape[-1])))
    whole = random_moe_weights(cfg, "cpu", gen, 0, 1, std=0.1, layer_seed=5)
    r, gu, dn = dense(whole)
    want = moe_reference(x, wq_pack.unpack_to_dense(r), gu, dn, 2)
    total = torch.zeros_like(want)
    for rank in range(4):                                               # 2 owners x 2 lanes
        part = random_moe_weights(cfg, "cpu", gen, rank, 4, std=0.1, layer_seed=5, ep_size=2)
        assert part.expert_count == 2 and part.expert_lo == (rank // 2) * 2 and part.gate_up.n == 256
        r, gu, dn = dense(part)
        total += moe_reference(x, wq_pack.unpack_to_dense(r), gu, dn, 2, expert_lo=part.expert_lo)
    assert float((total - want).norm() / want.norm()) < 5e-3
    with pytest.raises(ValueError):
        random_moe_weights(cfg, "cpu", gen, 0, 4, ep_size=1)            # 64-feature lanes: not whole groups


def _moe_dispatch_rank(rank, world, port, q):
    import torch.distributed as dist
    from cubic_serve_b200.models.distributed_reference import moe_dispatch_combine_reference
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(17)
    E, H, I, T = 8, 32, 48, 12
    router = (torch.randn(E, H, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = [(torch.randn(2 * I, H, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    down = [(torch.randn(H, I, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    per, rows = E // world, T // world
    y, sent = moe_dispatch_combine_reference(x[rank * rows:(rank + 1) * rows], router, gate_up[rank * per:(rank + 1) * per],
                                             down[rank * per:(rank + 1) * per], 3, dist.group.WORLD)
    q.put((rank, y, sent))
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharded_dispatch_and_combine_equals_the_single_process_block():
    """Rows live on their home rank, experts on their owners: every row travels once per owner it needs (never once per
    expert), comes back pre-summed, and the home rank's sum equals the block computed in one process."""
    from cubic_serve_b200.models.moe import moe_reference
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_moe_dispatch_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {r: (y, sent) for r, y, sent in (q.get(timeout=120) for _ in range(world))}
    for p in procs:
        p.join(timeout=60)
    g = torch.Generator().manual_seed(17)
    E, H, I, T = 8, 32, 48, 12
    router = (torch.randn(E, H, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = [(torch.randn(2 * I, H, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    down = [(torch.randn(H, I, generator=g) * 0.2).to(torch.bfloat16) for _ in range(E)]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    want = moe_reference(x, router, gate_up, down, 3)
    y = torch.cat([got[0][0], got[1][0]])
    assert float((y - want).norm() / want.norm()) < 1e-5
    for r in range(world):
        sent = got[r][1]
        # top-3 of 8 experts on 2 owners: a row needs one or two owners, never three transfers
        assert 6 <= sum(sent) <= 12 and max(sent) <= 6
