"""Two ranks on two GPUs: sequence-sharded decode through the fused NVLink exchange kernel
and through NCCL, both against the single-GPU result over the whole sequence; KV-head
sharding against the same.  Skipped unless at least two GPUs are visible."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import gqa_decode_b200 as G
    from gqa_decode_b200 import distributed as D

    g = torch.Generator().manual_seed(5)
    b, hq, hkv, d, s = 2, 64, 8, 128, 8192
    mk = lambda *sh: torch.randn(*sh, generator=g).to(torch.bfloat16)
    q, k, v = mk(b, hq, d), mk(b, hkv, s, d), mk(b, hkv, s, d)
    lens = [s, 3000]  # the second sequence ends inside the first shard
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    whole, whole32 = G.gqa_decode_attention_batched(q.to(dev), k.to(dev), v.to(dev), sl, return_f32=True)
    lo, hi = D.shard_range(s, world, rank)
    ks, vs = k[:, :, lo:hi].contiguous().to(dev), v[:, :, lo:hi].contiguous().to(dev)
    local_lens = torch.tensor([max(0, min(l, hi) - lo) for l in lens], dtype=torch.int32, device=dev)
    errs = {}
    ex = D.NvlinkExchange(b * hq, d, dev)
    for it in range(3):  # repeated exchanges reuse the buffers (epochs, parity halves)
        out = D.sequence_sharded_decode(q.to(dev), ks, vs, local_lens, exchange=ex)
    errs["nvlink"] = float((out.float() - whole.float()).abs().max())
    errs["nvlink_status"] = ex.check()
    out = D.sequence_sharded_decode(q.to(dev), ks, vs, local_lens)
    errs["nccl"] = float((out.float() - whole.float()).abs().max())
    qs, hs = D.shard_kv_heads(hq, hkv, world, rank)
    outh = D.head_sharded_decode(q[:, qs].contiguous().to(dev), k[:, hs].contiguous().to(dev),
                                 v[:, hs].contiguous().to(dev), sl, gather_output=True)
    errs["heads"] = float((outh.float() - whole.float()).abs().max())
    errs["status"] = G.read_status()
    torch.save(errs, os.path.join(result_dir, f"errs_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_sharded_decode(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        e = torch.load(os.path.join(tmp_path, f"errs_{r}.pt"))
        assert e["status"] == 0 and e["nvlink_status"] == 0, e
        # same partials, same merge arithmetic: shard results differ from the whole only by
        # float32 rounding, far below one bf16 ulp of the O(0.1) outputs
        assert e["nvlink"] < 2e-3 and e["nccl"] < 2e-3 and e["heads"] < 2e-3, e
