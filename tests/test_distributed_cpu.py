"""World-size-2 (and 3) runs of the sharded decode plumbing on CPU ranks (gloo).

The per-rank attention and the merge are injected from the CPU oracle here - this test
covers the sharding arithmetic, the message layout of the all-gather and the merge
order, not the CUDA kernels (tests/test_decode_gpu.py does that on one GPU)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_local(q, k, v, seq_lens, **kw):
    from oracle import gqa_oracle as O

    b, hq, d = q.shape
    o = torch.zeros(b, hq, d)
    lse = torch.full((b, hq), float("-inf"))
    for i in range(b):
        n = k.shape[2] if seq_lens is None else int(seq_lens[i])
        if n:
            o[i] = O.attend_one_sequence_f64(q[i], k[i, :, :n], v[i, :, :n]).float()
            lse[i] = O.lse_one_sequence(q[i], k[i, :, :n]).float()
    return o, lse


def _oracle_merge(o_parts, lse_parts, dtype):
    from oracle import gqa_oracle as O

    return O.merge_lse_partials(o_parts, lse_parts).to(dtype)


def _worker(rank, world, port, mode, result_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gqa_decode_b200 import distributed as D
    from oracle import gqa_oracle as O

    g = torch.Generator().manual_seed(5)
    b, hq, hkv, d, s = 2, 16, 4, 64, 301
    q = O.randn_bf16((b, hq, d), g)
    k = O.randn_bf16((b, hkv, s, d), g)
    v = O.randn_bf16((b, hkv, s, d), g)
    lens = [301, 120]  # second sequence ends inside the first shard(s): later shards are empty
    want = torch.stack([O.attend_one_sequence_f64(q[i], k[i, :, :lens[i]], v[i, :, :lens[i]]) for i in range(b)])
    if mode == "sequence":
        lo, hi = D.shard_range(s, world, rank)
        local_lens = torch.tensor([max(0, min(l, hi) - lo) for l in lens], dtype=torch.int32)
        out = D.sequence_sharded_decode(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(),
                                        local_lens, local_fn=_oracle_local, merge_fn=_oracle_merge)
    else:
        qs, ks = D.shard_kv_heads(hq, hkv, world, rank)

        def local(qq, kk, vv, sl, **kw):
            o, _ = _oracle_local(qq, kk, vv, sl)
            return o.to(qq.dtype)

        out = D.head_sharded_decode(q[:, qs].contiguous(), k[:, ks].contiguous(), v[:, ks].contiguous(),
                                    torch.tensor(lens, dtype=torch.int32), gather_output=True, local_fn=local)
    err = float((out.double() - want).abs().max())
    torch.save(err, os.path.join(result_dir, f"err_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode,world", [("sequence", 2), ("sequence", 3), ("heads", 2)])
def test_sharded_decode_gloo(tmp_path, mode, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, mode, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert torch.load(os.path.join(tmp_path, f"err_{r}.pt")) < 1.2e-2  # bf16 output rounding


def test_shard_helpers():
    from gqa_decode_b200 import distributed as D

    for total in (0, 1, 7, 131072):
        for world in (1, 2, 3, 8):
            cuts = [D.shard_range(total, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert max(e - b for b, e in cuts) - min(e - b for b, e in cuts) <= 1
    qs, ks = D.shard_kv_heads(64, 8, 4, 3)
    assert (qs, ks) == (slice(48, 64), slice(6, 8))
    with pytest.raises(ValueError):
        D.shard_kv_heads(64, 8, 3, 0)
    with pytest.raises(ValueError):
        D.shard_range(10, 2, 2)
