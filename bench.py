#!/usr/bin/env python
"""Benchmark of the GQA decode-attention step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Metric: achieved HBM throughput of one decode-attention step, in TB/s, with the
algorithmic bytes of the reference (2 * Hkv * S * D * bytes_per_element summed over the
sequences: K and V only), and the matching microseconds per step.

Workloads (synthetic, seeded; shapes of the five benchmark configurations):
  ragged         B=16 Hq=32 Hkv=8 D=128 bf16, lengths 1, 7, 32768 + 13 uniform in [1, 32768]
                 (default; every rank runs its own batch: weak scaling, no collective)
  single         B=1  Hq=32 Hkv=8 D=128 bf16 S=16384
  fp8            B=8  Hq=32 Hkv=8 D=128 E4M3 S=32768, 0.1 % outliers x20
  paged          config 2 with K/V in shuffled 64-row pages + block table
  seqshard       B=1  Hq=64 Hkv=8 D=128 bf16 S=131072 split into N contiguous sequence shards,
                 (O, LSE) all-gathered with NCCL and merged on device (strong scaling)
  headshard      B=64 Hq=64 Hkv=8 D=128 bf16 S=8192, KV heads split over N ranks (strong)
  headshard_fp8  same with E4M3 K/V

One step = one pass of the decode path over the batch.  `value` is measured with the
inputs resident in HBM; `e2e` is the same step driven from pinned host buffers with the
host->device copies of q/K/V and the device->host read of the output inside the timed
region.  `--impl reference` times the CPU restatement of the reference's PyTorch path
(oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# dram bytes moved per algorithmic byte, from the ncu capture summarised in
# profiles/decode_kernel_bf16_ragged.md and profiles/decode_kernel_fp8_batch8.md
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = {"bf16": 1.017, "e4m3": 1.011}
FALLBACK_HBM_GBS = 6650.0


# ----------------------------------------------------------------------------- workloads
def make_lengths(seed: int, batch: int = 16, max_len: int = 32768):
    g = torch.Generator().manual_seed(seed)
    rest = torch.randint(1, max_len + 1, (batch - 3,), generator=g).tolist()
    return [1, 7, max_len] + rest


class Workload:
    """Device-resident inputs of one rank plus the callable that runs one step."""

    def __init__(self, name: str, rank: int, world: int, dev: torch.device, batch: int = 16,
                 exchange: str = "fused", gather: str = "none", page_size: int = 64):
        import gqa_decode_b200 as G

        self.G, self.name, self.rank, self.world, self.dev = G, name, rank, world, dev
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        rn = lambda *s: torch.randn(*s, generator=gen, device=dev, dtype=torch.float32)
        self.fp8 = name in ("fp8", "headshard_fp8")
        self.scaling = "weak"
        self.launches_per_step = 1
        self.collective = None
        d = 128
        if name == "ragged":
            self.lens = make_lengths(1234 + rank, batch)
            hq, hkv = 32, 8
            rows = hkv * sum(self.lens)
            self.q = rn(batch, hq, d).to(torch.bfloat16)
            self.k = rn(rows, d).to(torch.bfloat16)
            self.v = rn(rows, d).to(torch.bfloat16)
            self.seq_lens = torch.tensor(self.lens, dtype=torch.int32, device=dev)
            self.kw = dict(layout="packed", max_seq_len=32768, num_kv_heads=hkv)
            self.desc = {"workload": "ragged_batch_decode(config 2)", "batch": batch, "num_q_heads": hq,
                         "num_kv_heads": hkv, "head_dim": d, "kv_dtype": "bf16",
                         "seq_lens": self.lens, "kv_layout": "packed", "parallelism": f"replica x{world}"}
        elif name == "paged":
            # config 2's ragged batch held the way serving engines hold it: a pool of
            # 64-row pages [pages, Hkv, 64, D] handed out in shuffled order, plus a block table
            self.lens = make_lengths(1234 + rank, batch)
            hq, hkv, page = 32, 8, page_size
            need = [(l + page - 1) // page for l in self.lens]
            pages = sum(need)
            self.q = rn(batch, hq, d).to(torch.bfloat16)
            self.k = rn(pages, hkv, page, d).to(torch.bfloat16)
            self.v = rn(pages, hkv, page, d).to(torch.bfloat16)
            order = torch.randperm(pages, generator=gen, device=dev).to(torch.int32)
            table = torch.zeros(batch, max(need), dtype=torch.int32, device=dev)
            at = 0
            for i, n in enumerate(need):
                table[i, :n] = order[at:at + n]
                at += n
            self.seq_lens = torch.tensor(self.lens, dtype=torch.int32, device=dev)
            self.kw = dict(layout="paged_hnd", block_table=table, max_seq_len=max(need) * page)
            self.desc = {"workload": "ragged_batch_decode(config 2), paged KV", "batch": batch,
                         "num_q_heads": hq, "num_kv_heads": hkv, "head_dim": d, "kv_dtype": "bf16",
                         "seq_lens": self.lens, "kv_layout": f"paged_hnd, {page} rows per page, shuffled",
                         "parallelism": f"replica x{world}"}
        elif name == "single":
            hq, hkv, s = 32, 8, 16384
            self.lens = [s]
            self.q = rn(1, hq, d).to(torch.bfloat16)
            # rotate through enough distinct K/V sets to exceed L2 several times
            self.nbuf = 10
            self.kbufs = [rn(1, hkv, s, d).to(torch.bfloat16) for _ in range(self.nbuf)]
            self.vbufs = [rn(1, hkv, s, d).to(torch.bfloat16) for _ in range(self.nbuf)]
            self.k, self.v = self.kbufs[0], self.vbufs[0]
            self.seq_lens, self.kw = None, {}
            self.desc = {"workload": "single_sequence_decode(config 1)", "batch": 1, "num_q_heads": hq,
                         "num_kv_heads": hkv, "head_dim": d, "kv_dtype": "bf16", "seq_len": s,
                         "kv_buffers_rotated": self.nbuf, "parallelism": f"replica x{world}"}
        elif name == "fp8":
            b, hq, hkv, s = 8, 32, 8, 32768
            self.lens = [s] * b
            self.q = rn(b, hq, d).to(torch.bfloat16)

            def outlier():
                x = rn(b, hkv, s, d)
                hit = torch.rand(x.shape, generator=gen, device=dev) < 1e-3
                return torch.where(hit, x * 20.0, x).to(torch.bfloat16)

            from gqa_decode_b200 import fp8_utils

            ks, vs, k8, v8 = [], [], [], []
            kk, vv = outlier(), outlier()
            for i in range(b):
                a, c, e, f = fp8_utils.quantize_kv_fp8(kk[i], vv[i])
                k8.append(a), v8.append(c), ks.append(e), vs.append(f)
            self.k, self.v = torch.stack(k8), torch.stack(v8)
            self.kw = dict(k_scale=torch.stack(ks), v_scale=torch.stack(vs))
            self.seq_lens = None
            del kk, vv
            self.desc = {"workload": "fp8_kv_decode(config 3)", "batch": b, "num_q_heads": hq,
                         "num_kv_heads": hkv, "head_dim": d, "kv_dtype": "e4m3", "seq_len": s,
                         "parallelism": f"replica x{world}"}
        elif name == "seqshard":
            hq, hkv, s = 64, 8, 131072
            assert s % world == 0
            self.scaling = "strong"
            self.lens = [s // world]
            gq = torch.Generator(device=dev).manual_seed(99)  # q identical on every rank
            self.q = torch.randn(1, hq, d, generator=gq, device=dev).to(torch.bfloat16)
            self.k = rn(1, hkv, s // world, d).to(torch.bfloat16)
            self.v = rn(1, hkv, s // world, d).to(torch.bfloat16)
            self.seq_lens, self.kw = None, {}
            self.collective = "all_gather(O fp32 [64,128] + LSE [64]) + on-device merge" if world > 1 else None
            self.launches_per_step = 2 if world > 1 else 1
            self.desc = {"workload": "long_context_sequence_sharded(config 4)", "batch": 1,
                         "num_q_heads": hq, "num_kv_heads": hkv, "head_dim": d, "kv_dtype": "bf16",
                         "seq_len": s, "parallelism": f"sp{world}"}
        elif name in ("headshard", "headshard_fp8"):
            b, hq, hkv, s = 64, 64, 8, 8192
            assert hkv % world == 0
            self.scaling = "strong"
            hkv_l, hq_l = hkv // world, hq // world
            self.lens = [s] * b
            self.q = rn(b, hq_l, d).to(torch.bfloat16)
            if self.fp8:
                self.k = rn(b, hkv_l, s, d).to(torch.float8_e4m3fn)
                self.v = rn(b, hkv_l, s, d).to(torch.float8_e4m3fn)
                sc = torch.full((b, hkv_l), 1.0 / 64, device=dev)
                self.kw = dict(k_scale=sc, v_scale=sc.clone())
            else:
                self.k = rn(b, hkv_l, s, d).to(torch.bfloat16)
                self.v = rn(b, hkv_l, s, d).to(torch.bfloat16)
                self.kw = {}
            self.seq_lens = None
            self.desc = {"workload": "batched_decode_kv_head_sharded(config 5)", "batch": b,
                         "num_q_heads": hq, "num_kv_heads": hkv, "head_dim": d,
                         "kv_dtype": "e4m3" if self.fp8 else "bf16", "seq_len": s,
                         "parallelism": f"tp{world} (KV heads, no collective)"}
        else:
            raise SystemExit(f"unknown workload {name}")
        hkv_local = self.k.shape[1] if self.k.dim() == 4 else 8
        esz = 1 if self.fp8 else 2
        self.bytes_per_step = 2 * hkv_local * sum(self.lens) * d * esz  # this rank, K + V only
        self.step_index = 0
        self.gather = gather if name in ("headshard", "headshard_fp8") and world > 1 else "none"
        self.head_gather = None
        if self.gather == "fused":
            from gqa_decode_b200.distributed import HeadGather

            self.head_gather = HeadGather(self.q.shape[0], self.q.shape[1], d, torch.bfloat16, dev)
            self.collective = "outputs gathered on every rank inside the decode kernel (peer stores + flags)"
            self.desc["parallelism"] = f"tp{world} (KV heads, fused output gather)"
        elif self.gather == "nccl":
            import torch.distributed as dist

            self.dist = dist
            self.collective = "NCCL all-gather of the bf16 outputs after the decode kernel"
            self.launches_per_step = 2
            self.gathered = torch.empty(world * self.q.shape[0], self.q.shape[1], d,
                                        dtype=torch.bfloat16, device=dev)
            self.desc["parallelism"] = f"tp{world} (KV heads, NCCL output all-gather)"
        self.exchange = None
        if name == "seqshard" and world > 1 and exchange == "nvlink":
            from gqa_decode_b200.distributed import NvlinkExchange

            self.exchange = NvlinkExchange(hq, d, dev)
            self.collective = "fused NVLink push + flag + merge kernel (peer stores, symmetric memory)"
        self.fused_exchange = None
        if name == "seqshard" and world > 1 and exchange == "fused":
            from gqa_decode_b200.distributed import FusedSequenceExchange

            self.fused_exchange = FusedSequenceExchange(1, hq, d, dev)
            self.collective = "exchange and merge inside the decode kernel (peer stores + flags, symmetric memory)"
            self.launches_per_step = 1
        if name == "seqshard" and world > 1:
            import torch.distributed as dist

            self.dist = dist
            self.gather_o = torch.empty(world * hq, d, dtype=torch.float32, device=dev)
            self.gather_l = torch.empty(world * hq, dtype=torch.float32, device=dev)

    def prepare(self):
        """Bind the steps once (validated argument blocks); `single` additionally captures
        each launch in a CUDA graph because a 67 MB step is shorter than a Python call."""
        G = self.G
        if self.name == "single":
            self.plans = [G.plan_decode(self.q, self.kbufs[i], self.vbufs[i], None) for i in range(self.nbuf)]
            for p in self.plans:
                p.run()
            torch.cuda.synchronize()
            self.graphs = []
            for p in self.plans:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    p.run()
                self.graphs.append(g)
            self.desc["launch"] = "one CUDA graph per K/V buffer set, replayed"
        elif self.fused_exchange is not None:
            self.fused_step = self.fused_exchange.plan(self.q, self.k, self.v, None)
        elif self.name == "seqshard" and self.world > 1:
            self.plan = G.plan_decode(self.q, self.k, self.v, None, return_f32=True, return_lse=True)
        elif self.head_gather is not None:
            self.gather_step = self.head_gather.plan(self.q, self.k, self.v, self.seq_lens, **self.kw)
        else:
            self.plan = G.plan_decode(self.q, self.k, self.v, self.seq_lens, **self.kw)

    def step(self):
        G = self.G
        if self.name == "single":
            i = self.step_index % self.nbuf
            self.step_index += 1
            self.graphs[i].replay()
            return self.plans[i].result
        if self.fused_exchange is not None:
            return self.fused_step()
        if self.name == "seqshard" and self.world > 1:
            _, o32, lse = self.plan.run()
            if self.exchange is not None:
                return self.exchange.merge(o32[0], lse[0], torch.bfloat16)
            self.dist.all_gather_into_tensor(self.gather_o, o32[0])
            self.dist.all_gather_into_tensor(self.gather_l, lse[0])
            w = self.world
            return G.merge_partials(self.gather_o.view(w, -1, 128), self.gather_l.view(w, -1),
                                    out_dtype=torch.bfloat16)
        if self.head_gather is not None:
            return self.gather_step()
        out = self.plan.run()
        if self.gather == "nccl":
            self.dist.all_gather_into_tensor(self.gathered, out)
            return self.gathered
        return out


# ----------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU every 50 ms (NVML, read-only)."""

    def __init__(self, dev_index: int):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.util = []
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(dev_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(dev_index)
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:  # pragma: no cover
            self.err = repr(e)

    NAMES = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
             0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._halt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                ut = nv.nvmlDeviceGetUtilizationRates(self.h).gpu
                mask = int(get(self.h))
                self.samples.append(mhz)
                self.util.append(ut)
                if ut > 0:
                    for bit, name in self.NAMES.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.05)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        busy = [m for m, u in zip(self.samples, self.util) if u > 0] or self.samples
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(busy)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_reference_step(sample):
    from oracle import gqa_oracle as O

    outs = []
    for q, k, v in sample:
        outs.append(O.attend_one_sequence(q, k, v))
    return outs


def make_cpu_sample(name: str, budget_keys: int):
    """A bounded sample of the workload for the CPU oracle: whole sequences of the batch,
    in order, up to about `budget_keys` keys in total."""
    from oracle import gqa_oracle as O

    g = torch.Generator().manual_seed(1234)
    if name in ("ragged", "paged"):
        lens, hq, hkv = make_lengths(1234), 32, 8
    elif name == "single":
        lens, hq, hkv = [16384], 32, 8
    elif name == "fp8":
        lens, hq, hkv = [32768] * 8, 32, 8
    elif name == "seqshard":
        lens, hq, hkv = [131072], 64, 8
    else:
        lens, hq, hkv = [8192] * 64, 64, 8
    sample, used, picked = [], 0, []
    for l in lens:
        if used and used + l > budget_keys:
            continue
        l_eff = min(l, budget_keys)
        q = O.randn_bf16((hq, 128), g)
        k = O.randn_bf16((hkv, l_eff, 128), g)
        v = O.randn_bf16((hkv, l_eff, 128), g)
        sample.append((q, k, v))
        picked.append(l_eff)
        used += l_eff
        if used >= budget_keys:
            break
    nbytes = 2 * hkv * used * 128 * 2  # the oracle attends over dequantised bf16 K/V
    return sample, nbytes, f"{len(picked)} sequences of the batch with KV lengths {picked} (bf16 K/V)"


def time_cpu(name: str, steps: int, warmup: int, budget_s: float):
    torch.set_num_threads(os.cpu_count() or 1)
    budget_keys = 40000
    sample, nbytes, what = make_cpu_sample(name, budget_keys)
    t = time.perf_counter()
    cpu_reference_step(sample)
    first = time.perf_counter() - t
    # shrink the sample if the whole run would not fit the budget
    while first * (steps + warmup) > budget_s and budget_keys > 2048:
        budget_keys //= 2
        sample, nbytes, what = make_cpu_sample(name, budget_keys)
        t = time.perf_counter()
        cpu_reference_step(sample)
        first = time.perf_counter() - t
    for _ in range(max(0, warmup - 1)):
        cpu_reference_step(sample)
    t = time.perf_counter()
    for _ in range(steps):
        cpu_reference_step(sample)
    dt = (time.perf_counter() - t) / steps
    return dt, nbytes, what


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="ragged",
                    choices=["ragged", "paged", "single", "fp8", "seqshard", "headshard", "headshard_fp8"])
    ap.add_argument("--page-size", type=int, default=64, help="paged workload: rows per page")
    ap.add_argument("--batch", type=int, default=16, help="ragged workload only: sequences per rank")
    ap.add_argument("--preheat-s", type=float, default=0.05,
                    help="seconds of untimed steps after the warm-up so the SM clock leaves its idle "
                         "state (0 for profiler runs).  Kept short: after about 0.3 s of continuous "
                         "streaming the B200s of this pool settle about 8 %% below their burst "
                         "bandwidth, and the roofline peak in MEASURED_PEAKS.json is a burst figure")
    ap.add_argument("--gather", default="none", choices=["none", "fused", "nccl"],
                    help="headshard at N>1: leave outputs sharded, gather them inside the decode kernel, "
                         "or all-gather them with NCCL afterwards")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nvlink", "nccl"],
                    help="seqshard at N>1: exchange+merge inside the decode kernel, a separate peer-store "
                         "exchange+merge kernel, or NCCL all-gather + merge")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", "29511",
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))

    base = {"metric": "decode_attn_achieved_hbm_throughput", "unit": "TB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "vs_baseline": None, "data": "synthetic"}

    if args.impl == "reference":
        if rank != 0:
            return
        dt, nbytes, what = time_cpu(args.workload, args.steps, max(1, args.warmup), budget_s=200.0)
        val = nbytes / dt / 1e12
        cores = torch.get_num_threads()
        line = dict(base)
        line.update({
            "impl": "reference", "value": val, "ms_per_step": dt * 1e3, "us_per_step": dt * 1e6,
            "scaling": "weak", "dtype": "f32",
            "config": {"workload": {"ragged": "ragged_batch_decode(config 2)"}.get(args.workload, args.workload),
                       "sample": what},
            "cpu_baseline": {"value": val, "unit": "TB/s", "cores": cores, "kind": "port", "sample": what},
            "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        })
        print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    from gqa_decode_b200 import _native

    _native.load()
    import gqa_decode_b200 as G

    wl = Workload(args.workload, rank, world, dev, args.batch, args.exchange, args.gather, args.page_size)
    wl.prepare()
    sampler = ClockSampler(local_rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up: W steps plus a short run so the SM clock is at its loaded level.  The number of
    # extra steps is agreed between the ranks (steps with an exchange are collective: every
    # rank must run the same count), from the slowest rank's estimate of a step.
    for _ in range(max(3, args.warmup)):
        wl.step()
    torch.cuda.synchronize()
    sampler.start()
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record()
    for _ in range(5):
        wl.step()
    w1.record()
    torch.cuda.synchronize()
    est_ms = max(w0.elapsed_time(w1) / 5, 1e-3)
    extra = torch.tensor([min(int(args.preheat_s * 1e3 / est_ms) + 1, 100000) if args.preheat_s > 0 else 0],
                         device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(extra, op=dist.ReduceOp.MAX)
    for _ in range(int(extra.item())):
        wl.step()
    torch.cuda.synchronize()

    # ---- device-resident timing
    barrier()
    # one event pair around the K steps: an event after every launch would keep launch
    # k+1 from starting while launch k drains
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        wl.step()
    ev1.record()
    barrier()
    total_ms = ev0.elapsed_time(ev1)
    per_step_ms = [total_ms / args.steps]
    status = G.read_status()

    # ---- end to end from pinned host buffers
    e2e = None
    if not args.no_e2e and args.workload != "single":
        host = {n: getattr(wl, n).cpu().pin_memory() for n in ("q", "k", "v")}
        out_host = torch.empty(wl.q.shape, dtype=torch.bfloat16).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = out_host.numel() * out_host.element_size()
        n_e2e = max(3, min(args.steps, 20))

        def e2e_step():
            wl.q.copy_(host["q"], non_blocking=True)
            wl.k.copy_(host["k"], non_blocking=True)
            wl.v.copy_(host["v"], non_blocking=True)
            out = wl.step()
            out_host.copy_(out.view(out_host.shape), non_blocking=True)

        e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        barrier()
        e2e_ms = a.elapsed_time(b) / n_e2e
        e2e = (e2e_ms, h2d, d2h, n_e2e)
    clocks = sampler.stop()

    # ---- reduce over ranks: max time, sum bytes
    t = torch.tensor([total_ms, e2e[0] if e2e else 0.0], device=dev, dtype=torch.float64)
    nb = torch.tensor([float(wl.bytes_per_step)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nb, op=dist.ReduceOp.SUM)
    total_ms_max, e2e_ms_max = t.tolist()
    job_bytes = nb.item()

    if rank == 0:
        ms_per_step = total_ms_max / args.steps
        value = job_bytes / (ms_per_step * 1e-3) / 1e12
        peak = FALLBACK_HBM_GBS
        peak_src = "fallback"
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak = float(json.load(f)["hbm_gbs"])
                peak_src = "measured"
        except Exception:
            pass
        kern_ms = statistics.mean(per_step_ms)
        achieved = wl.bytes_per_step / (kern_ms * 1e-3) / 1e9
        ratio = DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE["e4m3" if wl.fp8 else "bf16"]
        line = dict(base)
        cfg = dict(wl.desc)
        cfg.update({"l2": "inputs larger than L2 (126 MB), read with an evict-first policy"
                    if wl.bytes_per_step > 4 * 126e6 or args.workload == "single"
                    else "inputs may partly fit L2",
                    "algorithmic_bytes_per_step": int(job_bytes), "kernel_status": status,
                    "preheat": f"{args.preheat_s} s of untimed steps after the warm-up"})
        if wl.collective:
            cfg["collective"] = wl.collective
        line.update({
            "value": value, "ms_per_step": ms_per_step, "us_per_step": ms_per_step * 1e3,
            "scaling": wl.scaling, "dtype": "e4m3->bf16 mma, f32 accumulate" if wl.fp8 else "bf16 mma, f32 accumulate",
            "config": cfg,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_src + " (MEASURED_PEAKS.json hbm_gbs)",
                         "traffic": None if ratio is None else ratio * wl.bytes_per_step,
                         "kernel": "gqa::decode_kernel", "avg_launch_ms": kern_ms,
                         "frac_of_nominal_8TBps": achieved / 8000.0},
            "clocks": clocks,
            "gpu_launches": args.steps * wl.launches_per_step,
        })
        if e2e:
            line["e2e"] = {"value": job_bytes / (e2e_ms_max * 1e-3) / 1e12, "unit": "TB/s",
                           "ms_per_step": e2e_ms_max, "steps": e2e[3],
                           "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2]}
        if world == 1 and not args.no_cpu:
            dt, nbytes, what = time_cpu(args.workload, steps=2, warmup=1, budget_s=25.0)
            line["cpu_baseline"] = {"value": nbytes / dt / 1e12, "unit": "TB/s",
                                    "cores": torch.get_num_threads(), "kind": "port", "sample": what,
                                    "ms_per_sample": dt * 1e3}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
