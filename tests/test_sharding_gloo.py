"""CPU, world_size 2 over gloo: the multi-GPU path shards (batch, KV-head group) units without any
data-path collective; ranks only agree on the step time and gather per-shard check results."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "gemm4-attention-kernels_b200"))
    sys.path.insert(0, root)
    from splitd_flash_attn import sharding as S

    from oracle import attention_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, Sq, Hq, Hkv, D = 2, 24, 8, 4, 512
    gen = torch.Generator().manual_seed(0)  # identical data on every rank
    q = torch.randn(B, Sq, Hq, D, generator=gen)
    k = torch.randn(B, Sq, Hkv, D, generator=gen)
    v = torch.randn(B, Sq, Hkv, D, generator=gen)
    full, _ = O.attention_fwd(q, k, v, True)
    shards = S.layer_shards(B, Hkv)
    mine = S.shards_of_rank(len(shards), rank, world)
    local = {}
    for i in mine:
        qs, ks, vs = S.shard_views(q, k, v, shards[i], Hq, Hkv)
        o, _ = O.attention_fwd(qs, ks, vs, True)
        b, g = shards[i]
        local[i] = float((o[0] - full[b, :, g * 2 : (g + 1) * 2]).abs().max())
    errs = S.gather_shard_results(local, len(shards), "cpu")
    tmax = S.max_over_ranks(float(rank + 1), "cpu")
    if rank == 0:
        ret["errs"] = errs
        ret["tmax"] = tmax
        ret["mine"] = mine
    dist.destroy_process_group()


def test_shards_cover_the_layer_once():
    from splitd_flash_attn import sharding as S

    for world in (1, 2, 4, 8):
        seen = sorted(i for r in range(world) for i in S.shards_of_rank(8, r, world))
        assert seen == list(range(8))
    assert S.layer_shards(2, 4)[5] == (1, 1)


def test_two_ranks_gloo():
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret["mine"] == [0, 2, 4, 6]
        assert len(ret["errs"]) == 8 and max(ret["errs"]) < 1e-5  # sharded == unsharded, every shard reported
        assert ret["tmax"] == 2.0
