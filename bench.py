#!/usr/bin/env python
"""Benchmark of the GQA decode-attention step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Metric: achieved HBM throughput of one decode-attention step, in TB/s, with the
algorithmic bytes of the reference (2 * Hkv * S * D * bytes_per_element summed over the
sequences: K and V only, analysis/roofline.py:13-15 of the reference), and the matching
microseconds per step.

Workloads (synthetic, seeded; the shapes of the five benchmark configurations):
  headshard      B=64 Hq=64 Hkv=8 D=128 bf16 S=8192, KV heads (with their 8 query heads) split
                 over the N ranks, no collective: strong scaling.  The default, and the largest
                 configuration that fits one GPU.
  headshard_fp8  the same with E4M3 K/V
  single         B=1  Hq=32 Hkv=8 D=128 bf16 S=16384 (every rank a replica)
  ragged         B=16 Hq=32 Hkv=8 D=128 bf16, lengths 1, 7, 32768 + 13 uniform in [1, 32768]
                 (every rank a replica with the same lengths)
  fp8            B=8  Hq=32 Hkv=8 D=128 E4M3 S=32768, 0.1 % outliers x20 (replicas)
  paged          the ragged batch with K/V in shuffled pages + a block table (replicas)
  seqshard       B=1  Hq=64 Hkv=8 D=128 bf16 S=131072 split into N contiguous key ranges, the
                 partial (O, LSE) exchanged over NVLink and merged on device: strong scaling

One step = one pass of the decode path over the batch.  `value` is measured with the inputs
resident in HBM; `e2e` is the same step driven from pinned host buffers with the host->device
copies of q/K/V and the device->host read of the output inside the timed region.  After the
main workload the line gets an `others` object: the remaining workloads timed briefly at the
same N, each with its own fraction of the roofline, kernel status, a sustained figure and a
parity check of the step's output against the CPU oracle (outside every timed region).

`--impl reference` times the reference's own PyTorch path on the host cores (imported from
baseline/_ref when it is installed there, else its CPU restatement in oracle/) on a bounded
sample of the same workload: the very sequences the GPU arm holds at those positions.
"""
from __future__ import annotations

import argparse
import json
import math
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

# DRAM bytes moved per algorithmic byte of the decode kernel, from ncu captures
# (dram__bytes_read.sum + dram__bytes_write.sum over K+V bytes) on 537 MB launches, where the
# traffic is in proportion to the keys streamed: bf16 (one sequence of 131072 keys) 1.011,
# E4M3 (eight sequences of 32768 keys) 1.008
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = {"bf16": 1.011, "e4m3": 1.008}
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6
WORKLOADS = ["headshard", "headshard_fp8", "single", "ragged", "fp8", "paged", "seqshard"]
D = 128


# ----------------------------------------------------------------------------- shapes
def make_lengths(seed: int, batch: int = 16, max_len: int = 32768):
    g = torch.Generator().manual_seed(seed)
    rest = torch.randint(1, max_len + 1, (batch - 3,), generator=g).tolist()
    return [1, 7, max_len] + rest


def shape_of(name: str, batch: int = 16):
    """(sequence lengths, Hq, Hkv, E4M3?) of a workload, before any sharding."""
    if name in ("ragged", "paged"):
        return make_lengths(1234, batch), 32, 8, False
    if name == "single":
        return [16384], 32, 8, False
    if name == "fp8":
        return [32768] * 8, 32, 8, True
    if name == "seqshard":
        return [131072], 64, 8, False
    if name in ("headshard", "headshard_fp8"):
        return [8192] * 64, 64, 8, name.endswith("fp8")
    raise SystemExit(f"unknown workload {name}")


def rank_bytes(name: str, world: int, batch: int = 16) -> int:
    """Algorithmic bytes (K + V) one rank reads per step."""
    lens, _, hkv, fp8 = shape_of(name, batch)
    total = 2 * hkv * sum(lens) * D * (1 if fp8 else 2)
    return total // world if name in ("headshard", "headshard_fp8", "seqshard") else total


def kv_sets(name: str, world: int, batch: int = 16) -> int:
    """Distinct K/V sets a rank rotates through so that consecutive steps cannot be served
    from L2: one if a step reads more than four times the L2, else enough to exceed that."""
    b = rank_bytes(name, world, batch)
    return 1 if b >= 4 * L2_BYTES else int(math.ceil(4 * L2_BYTES / b))


def static_config(name: str, world: int, batch: int = 16, page_size: int = 64, gather: str = "none",
                  page_order: str = "shuffled") -> dict:
    """The description both arms print as `config`: the workload, its shape, how it is split
    and how the timing keeps L2 out of the picture."""
    lens, hq, hkv, fp8 = shape_of(name, batch)
    cfg = {"workload": {
        "headshard": "batched_decode_kv_head_sharded(config 5, bf16)",
        "headshard_fp8": "batched_decode_kv_head_sharded(config 5, e4m3)",
        "single": "single_sequence_decode(config 1)",
        "ragged": "ragged_batch_decode(config 2)",
        "paged": "ragged_batch_decode(config 2), paged KV",
        "fp8": "fp8_kv_decode(config 3)",
        "seqshard": "long_context_sequence_sharded(config 4)"}[name],
        "batch": len(lens), "num_q_heads": hq, "num_kv_heads": hkv, "head_dim": D,
        "kv_dtype": "e4m3" if fp8 else "bf16"}
    if len(set(lens)) == 1:
        cfg["seq_len"] = lens[0]
    else:
        cfg["seq_lens"] = lens
    if name in ("headshard", "headshard_fp8"):
        how = {"none": "no collective", "fused": "outputs gathered in-kernel", "nccl": "NCCL output all-gather"}
        cfg["parallelism"] = f"tp{world} (KV heads with their query groups; {how[gather if world > 1 else 'none']})"
    elif name == "seqshard":
        cfg["parallelism"] = f"sp{world} (contiguous key ranges; partial (O, LSE) exchanged and merged)"
    else:
        cfg["parallelism"] = f"replica x{world}"
    if name == "paged":
        cfg["kv_layout"] = f"paged_hnd, {page_size} rows per page, {page_order}"
    elif name == "ragged":
        cfg["kv_layout"] = "packed"
    n = kv_sets(name, world, batch)
    cfg["l2"] = ("inputs larger than L2 (126 MB), read with an evict-first policy" if n == 1 else
                 f"{n} K/V sets of {rank_bytes(name, world, batch) / 1e6:.0f} MB rotated (more than 4 x the 126 MB L2)")
    if name == "single":
        cfg["launch"] = f"one CUDA graph of {n} steps (one per K/V set), replayed"
    return cfg


# ----------------------------------------------------------------------------- seeded sample
# A few whole sequences of every workload come from the CPU generator, keyed by (workload,
# sequence, KV head): the GPU arm holds them at those positions of its first K/V set, the CPU
# arm times the reference on exactly them, and the parity check compares the two.
def sample_indices(name: str, batch: int = 16):
    lens, _, _, _ = shape_of(name, batch)
    if name in ("ragged", "paged"):
        return [i for i, l in enumerate(lens) if l <= 2048 or l == 32768][:4]
    if name in ("headshard", "headshard_fp8"):
        return [0, 1, 2, 3]
    return [0]


def sample_heads(name: str):
    """KV heads of the sampled sequences that are seeded on the CPU (all, except for the long
    sequence of config 4 where two heads keep the oracle's cost bounded)."""
    return [0, 1] if name == "seqshard" else list(range(8))


def sample_head(name: str, seq: int, head: int, length: int, group: int):
    """q [G, D], k [S, D], v [S, D] bf16 of one (sequence, KV head) of the seeded sample."""
    tag = WORKLOADS.index("headshard" if name == "headshard_fp8" else ("ragged" if name == "paged" else name))
    g = torch.Generator().manual_seed(77_000_000 + tag * 1_000_000 + seq * 1000 + head)
    mk = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)
    q, k, v = mk(group, D), mk(length, D), mk(length, D)
    if name == "fp8":  # config 3: 0.1 % of the elements scaled x20
        k = torch.where(torch.rand(k.shape, generator=g) < 1e-3, k * 20.0, k)
        v = torch.where(torch.rand(v.shape, generator=g) < 1e-3, v * 20.0, v)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def sample_sequence(name: str, seq: int, heads=None, batch: int = 16):
    """q [len(heads) * G, D], k/v [len(heads), S, D] bf16 of one sampled sequence."""
    lens, hq, hkv, _ = shape_of(name, batch)
    heads = sample_heads(name) if heads is None else heads
    parts = [sample_head(name, seq, h, lens[seq], hq // hkv) for h in heads]
    return (torch.cat([p[0] for p in parts]), torch.stack([p[1] for p in parts]),
            torch.stack([p[2] for p in parts]))


HEADSHARD_FP8_SCALE = 1.0 / 64


def quantize_sample(name: str, k: torch.Tensor, v: torch.Tensor, quantize):
    """E4M3 codes and per-head scales of a sampled sequence, as the GPU arm holds them:
    config 3 through the reference's quantize_kv_fp8 scheme (`quantize`), config 5 as a plain
    cast under a fixed scale."""
    if name == "fp8":
        return quantize(k, v)
    sc = torch.full((k.shape[0],), HEADSHARD_FP8_SCALE)
    return k.to(torch.float8_e4m3fn), v.to(torch.float8_e4m3fn), sc, sc.clone()


# ----------------------------------------------------------------------------- workloads
class Workload:
    """Device-resident inputs of one rank, the bound steps, and the parity check."""

    def __init__(self, name, rank, world, dev, batch=16, exchange="fused", gather="none", page_size=64,
                 dependent_launch=True, page_order="shuffled"):
        import gqa_decode_b200 as G

        self.G, self.name, self.rank, self.world, self.dev = G, name, rank, world, dev
        self.batch, self.page_size, self.pdl = batch, page_size, dependent_launch
        self.page_order = page_order
        lens, hq, hkv, self.fp8 = shape_of(name, batch)
        self.desc = static_config(name, world, batch, page_size, gather, page_order)
        self.scaling = "strong" if name in ("headshard", "headshard_fp8", "seqshard") else "weak"
        self.launches_per_step = 1
        self.collective = None
        self.group = hq // hkv
        # ---- this rank's share
        self.heads = list(range(hkv))           # global KV heads held here
        self.lens = list(lens)                  # keys per sequence held here
        self.key0 = 0                           # first key of every sequence held here
        if name in ("headshard", "headshard_fp8"):
            assert hkv % world == 0
            per = hkv // world
            self.heads = list(range(rank * per, (rank + 1) * per))
        elif name == "seqshard":
            assert lens[0] % world == 0
            self.lens = [lens[0] // world]
            self.key0 = rank * self.lens[0]
        self.hq_l, self.hkv_l = len(self.heads) * self.group, len(self.heads)
        esz = 1 if self.fp8 else 2
        self.bytes_per_step = 2 * self.hkv_l * sum(self.lens) * D * esz  # this rank, K + V only
        assert self.bytes_per_step == rank_bytes(name, world, batch)
        self.nbuf = kv_sets(name, world, batch)
        self.gather_mode = gather if name in ("headshard", "headshard_fp8") and world > 1 else "none"
        self.exchange_mode = exchange if name == "seqshard" and world > 1 else "none"
        self._generate()
        self._bind()

    # ---- inputs -----------------------------------------------------------------------
    def _randn(self, shape, seed):
        g = torch.Generator(device=self.dev).manual_seed(seed)
        return torch.randn(shape, generator=g, device=self.dev, dtype=torch.float32)

    def _generate(self):
        name, dev, B = self.name, self.dev, len(self.lens)
        packed = name in ("ragged", "paged")
        self.sets = []
        # replicas draw different bulk data per rank; shards are keyed by what they hold
        salt = self.rank if self.scaling == "weak" else 0
        for s in range(self.nbuf):
            seed = 5_000_000 + 10_000 * s + 100 * salt
            if packed:
                rows = self.hkv_l * sum(self.lens)
                k = self._randn((rows, D), seed + 1).to(torch.bfloat16)
                v = self._randn((rows, D), seed + 2).to(torch.bfloat16)
            else:
                S = self.lens[0]
                k = torch.empty(B, self.hkv_l, S, D, dtype=torch.bfloat16, device=dev)
                v = torch.empty_like(k)
                for j, h in enumerate(self.heads):  # keyed by the global head (and key range)
                    k[:, j] = self._randn((B, S, D), seed + 10 * h + 1 + 1000 * self.key0).to(torch.bfloat16)
                    v[:, j] = self._randn((B, S, D), seed + 10 * h + 2 + 1000 * self.key0).to(torch.bfloat16)
            self.sets.append([k, v, None, None])
        self.q = torch.empty(B, self.hq_l, D, dtype=torch.bfloat16, device=dev)
        for j, h in enumerate(self.heads):
            self.q[:, j * self.group:(j + 1) * self.group] = self._randn((B, self.group, D), 4_000_000 + h + 100 * salt).to(torch.bfloat16)
        if name == "fp8":  # bulk outliers, like the sample
            for st in self.sets:
                for t, sd in ((0, 31), (1, 32)):
                    hit = torch.rand(st[t].shape, generator=torch.Generator(device=dev).manual_seed(sd), device=dev) < 1e-3
                    st[t] = torch.where(hit, st[t] * 20.0, st[t])
        # ---- the seeded sample goes into set 0
        self.sample = {}  # seq -> (q [hq_l, D], k, v [hkv_l, S_local, D]) bf16 CPU tensors, or None per head
        k0, v0 = self.sets[0][0], self.sets[0][1]
        seeded = [h for h in self.heads if h in sample_heads(name)]
        offs = [0]
        for l in self.lens:
            offs.append(offs[-1] + self.hkv_l * l)
        for seq in sample_indices(name, self.batch):
            for h in seeded:
                j = self.heads.index(h)
                full = shape_of(name, self.batch)[0][seq]
                qh, kh, vh = sample_head(name, seq, h, full, self.group)
                kh, vh = kh[self.key0:self.key0 + self.lens[seq]], vh[self.key0:self.key0 + self.lens[seq]]
                self.q[seq, j * self.group:(j + 1) * self.group] = qh.to(dev)
                if packed:
                    r0 = offs[seq] + j * self.lens[seq]
                    k0[r0:r0 + self.lens[seq]] = kh.to(dev)
                    v0[r0:r0 + self.lens[seq]] = vh.to(dev)
                else:
                    k0[seq, j], v0[seq, j] = kh.to(dev), vh.to(dev)
        # ---- E4M3 caches
        if self.fp8:
            from gqa_decode_b200 import fp8_utils

            for st in self.sets:
                kb, vb = st[0], st[1]
                if name == "fp8":
                    quant = [fp8_utils.quantize_kv_fp8(kb[i], vb[i]) for i in range(B)]
                    st[0], st[1] = torch.stack([x[0] for x in quant]), torch.stack([x[1] for x in quant])
                    st[2], st[3] = torch.stack([x[2] for x in quant]), torch.stack([x[3] for x in quant])
                else:
                    st[0], st[1] = kb.to(torch.float8_e4m3fn), vb.to(torch.float8_e4m3fn)
                    st[2] = torch.full((B, self.hkv_l), HEADSHARD_FP8_SCALE, device=dev)
                    st[3] = st[2].clone()
                del kb, vb
        # ---- layouts
        self.kw, self.seq_lens = {}, None
        if packed:
            self.seq_lens = torch.tensor(self.lens, dtype=torch.int32, device=dev)
            self.kw = dict(layout="packed", max_seq_len=32768, num_kv_heads=self.hkv_l)
        if name == "paged":
            page = self.page_size
            need = [(l + page - 1) // page for l in self.lens]
            pages = sum(need)
            g = torch.Generator(device=dev).manual_seed(99)
            order = torch.randperm(pages, generator=g, device=dev).to(torch.int32)
            if self.page_order == "sequential":  # every sequence's pages in order, one after the other
                order = torch.arange(pages, device=dev, dtype=torch.int32)
            table = torch.zeros(B, max(need), dtype=torch.int32, device=dev)
            at = 0
            for i, n in enumerate(need):
                table[i, :n] = order[at:at + n]
                at += n
            for st in self.sets:  # scatter the packed rows into their pages
                pk = torch.zeros(pages, self.hkv_l, page, D, dtype=torch.bfloat16, device=dev)
                pv = torch.zeros_like(pk)
                for i, l in enumerate(self.lens):
                    ks = st[0][offs[i]:offs[i + 1]].view(self.hkv_l, l, D)
                    vs = st[1][offs[i]:offs[i + 1]].view(self.hkv_l, l, D)
                    for p in range(need[i]):
                        n = min(page, l - p * page)
                        pg = int(table[i, p])
                        pk[pg, :, :n] = ks[:, p * page:p * page + n]
                        pv[pg, :, :n] = vs[:, p * page:p * page + n]
                st[0], st[1] = pk, pv
            self.kw = dict(layout="paged_hnd", block_table=table, max_seq_len=max(need) * page)
        torch.cuda.synchronize(dev)

    # ---- steps ------------------------------------------------------------------------
    def _bind(self):
        """One pre-validated step per K/V set (a step is then one C call); all steps of a
        workload share one workspace, since they never overlap."""
        G, name, world = self.G, self.name, self.world
        self.step_index = 0
        self.graph = None
        opts = dict(self.kw, dependent_launch=self.pdl)
        B = len(self.lens)
        need = G.workspace_bytes(B, self.hq_l, self.hkv_l, D)
        ws = torch.zeros(need, dtype=torch.uint8, device=self.dev)
        self.steps, self.outputs, self.status_fns = [], [], []
        if self.gather_mode == "fused":
            from gqa_decode_b200.distributed import HeadGather

            self.hand_off = HeadGather(B, self.hq_l, D, torch.bfloat16, self.dev)
            self.collective = "outputs gathered on every rank inside the decode kernel (peer stores + flags over NVLink)"
        elif self.gather_mode == "nccl":
            import torch.distributed as dist

            self.collective = "NCCL all-gather of the bf16 outputs after the decode kernel"
            self.launches_per_step = 2
            gathered = torch.empty(world * B, self.hq_l, D, dtype=torch.bfloat16, device=self.dev)
        if self.exchange_mode == "fused":
            from gqa_decode_b200.distributed import FusedSequenceExchange

            self.hand_off = FusedSequenceExchange(B, self.hq_l, D, self.dev)
            self.collective = "exchange and merge inside the decode kernel (peer stores + flags over NVLink, symmetric memory)"
        elif self.exchange_mode == "nvlink":
            from gqa_decode_b200.distributed import NvlinkExchange

            exch = NvlinkExchange(B * self.hq_l, D, self.dev)
            self.collective = "decode kernel, then one peer-store exchange + merge kernel (symmetric memory)"
            self.launches_per_step = 2
        elif self.exchange_mode == "nccl":
            import torch.distributed as dist

            self.collective = "decode kernel, NCCL all-gather of O fp32 and LSE, merge kernel"
            self.launches_per_step = 4
            go = torch.empty(world * B * self.hq_l, D, dtype=torch.float32, device=self.dev)
            gl = torch.empty(world * B * self.hq_l, dtype=torch.float32, device=self.dev)
        for k, v, ks, vs in self.sets:
            sc = dict(k_scale=ks, v_scale=vs) if self.fp8 else {}
            if self.gather_mode == "fused" or self.exchange_mode == "fused":
                run = self.hand_off.plan(self.q, k, v, self.seq_lens, workspace=ws, **sc, **opts)
                self.steps.append(run)
                self.status_fns.append(run.status)
                continue
            want32 = self.exchange_mode in ("nvlink", "nccl")
            plan = G.plan_decode(self.q, k, v, self.seq_lens, workspace=ws, return_f32=want32,
                                 return_lse=want32, **sc, **opts)
            self.status_fns.append(plan.status)
            if self.exchange_mode == "nvlink":
                def run(plan=plan):
                    _, o32, lse = plan.run()
                    return exch.merge(o32.view(-1, D), lse.view(-1), torch.bfloat16).view(B, -1, D)
            elif self.exchange_mode == "nccl":
                def run(plan=plan):
                    _, o32, lse = plan.run()
                    dist.all_gather_into_tensor(go, o32.view(-1, D))
                    dist.all_gather_into_tensor(gl, lse.view(-1))
                    return G.merge_partials(go.view(world, -1, D), gl.view(world, -1),
                                            out_dtype=torch.bfloat16).view(B, -1, D)
            elif self.gather_mode == "nccl":
                def run(plan=plan):
                    dist.all_gather_into_tensor(gathered, plan.run())
                    return gathered.view(world, B, self.hq_l, D).permute(1, 0, 2, 3).reshape(B, -1, D)
            else:
                run = plan.run
            self.steps.append(run)
        if name == "single":
            # a 67 MB step is shorter than a Python call: the whole rotation of K/V sets is one
            # CUDA graph (its launches chained by programmatic dependent launch)
            for r in self.steps:
                r()
            torch.cuda.synchronize(self.dev)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                for r in self.steps:
                    self.last = r()

    def run_steps(self, n: int):
        """n steps, rotating through the K/V sets."""
        i = 0
        while i < n:
            at = self.step_index % self.nbuf
            if self.graph is not None and at == 0 and n - i >= self.nbuf:
                self.graph.replay()
                i += self.nbuf
                self.step_index += self.nbuf
                continue
            self.last = self.steps[at]()
            i += 1
            self.step_index += 1
        return self.last

    def run_set0(self):
        self.step_index = 1
        self.last = self.steps[0]()
        return self.last

    def status(self) -> int:
        st = 0
        for f in self.status_fns[:1]:  # the steps share one workspace
            st |= f()
        return st

    # ---- parity -----------------------------------------------------------------------
    def parity(self):
        """Largest |out - oracle| / (2e-2 + 1e-2 |oracle|) over the seeded sample after one
        step on K/V set 0 (a collective step where the workload has an exchange: every rank
        calls this; rank 0 evaluates).  The oracle is the C restatement of the reference's
        attention (float64), fed the sample's own CPU tensors."""
        out = self.run_set0()
        torch.cuda.synchronize(self.dev)
        if self.rank != 0:
            return None
        from oracle import c_oracle
        from oracle import gqa_oracle as O

        name = self.name
        seeded = sample_heads(name)
        worst, checked = 0.0, 0
        full_heads = list(range(8)) if (self.gather_mode != "none" or self.exchange_mode != "none") else self.heads
        heads = [h for h in full_heads if h in seeded]
        if self.gather_mode != "none":
            heads = [h for h in heads if h in self.heads or h == (self.heads[-1] + 1) % 8]  # own + one foreign head
        for seq in sample_indices(name, self.batch):
            q, k, v = sample_sequence(name, seq, heads, self.batch)
            ks = vs = None
            if self.fp8:
                k, v, ks, vs = quantize_sample(name, k, v, O.quantize_kv_e4m3)
                if name == "fp8":  # the scales are those of the whole sequence held on the GPU
                    ks, vs = self.sets[0][2][seq].cpu()[heads], self.sets[0][3][seq].cpu()[heads]
            ref, _ = c_oracle.attend(q, k, v, ks, vs)
            rows = torch.cat([out[seq, self._row0(h):self._row0(h) + self.group] for h in heads]).cpu()
            dlt = (rows.double() - ref).abs()
            worst = max(worst, float((dlt / (2e-2 + 1e-2 * ref.abs())).max()))
            checked += rows.shape[0]
        return {"max_err_over_tol": worst, "rows_checked": checked,
                "against": "oracle/gqa_oracle.c (float64) on the CPU-seeded sample sequences; tolerance 2e-2 + 1e-2 |ref|"}

    def _row0(self, h):
        """Row of global KV head h's first query head in this rank's step output."""
        if self.gather_mode != "none" or self.exchange_mode != "none":
            return h * self.group  # all heads are present in the output
        return self.heads.index(h) * self.group


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
def load_reference():
    """(attend, dequantize, quantize, kind): the reference's own functions when its package
    is installed under baseline/_ref (it needs the CuTe-DSL packages to import), else their
    CPU restatement in oracle/."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref_dir, "gqa_decode")) and "gqa_decode" not in sys.modules:
        sys.path.insert(0, ref_dir)
        try:
            import gqa_decode as R  # the reference package (first on the path)
            from gqa_decode import fp8_utils as RF

            if os.path.dirname(os.path.abspath(R.__file__)).startswith(ref_dir):
                return R.reference_gqa_decode, RF.dequantize_kv_fp8, RF.quantize_kv_fp8, "reference"
        except Exception:
            pass
        finally:
            sys.path.remove(ref_dir)
        for m in [m for m in sys.modules if m == "gqa_decode" or m.startswith("gqa_decode.")]:
            del sys.modules[m]
    from oracle import gqa_oracle as O

    return O.attend_one_sequence, O.dequantize_kv_e4m3, O.quantize_kv_e4m3, "port"


def time_cpu(name: str, steps: int, warmup: int, budget_s: float, batch: int = 16):
    """Time the reference's PyTorch path on whole sequences of the seeded sample, as many as
    fit the time budget.  Returns (seconds per step, algorithmic bytes per step, what, kind)."""
    torch.set_num_threads(os.cpu_count() or 1)
    attend, dequantize, quantize, kind = load_reference()
    lens, hq, hkv, fp8 = shape_of(name, batch)
    heads = sample_heads(name)
    seqs = []
    for seq in sample_indices(name, batch):
        q, k, v = sample_sequence(name, seq, heads, batch)
        if fp8:
            seqs.append((seq, q) + tuple(quantize_sample(name, k, v, quantize)))
        else:
            seqs.append((seq, q, k, v))

    def step(items):
        for it in items:
            if fp8:
                kd, vd = dequantize(it[2], it[3], it[4], it[5])
                attend(it[1], kd, vd)
            else:
                attend(it[1], it[2], it[3])

    use = seqs[:1]
    t = time.perf_counter()
    step(use)
    first = time.perf_counter() - t
    # take more sequences of the sample while the whole run stays inside the budget
    while len(use) < len(seqs) and first * (len(use) + 1) * (steps + warmup) < budget_s:
        use = seqs[:len(use) + 1]
    for _ in range(max(0, warmup - 1)):
        step(use)
    t = time.perf_counter()
    for _ in range(steps):
        step(use)
    dt = (time.perf_counter() - t) / steps
    keys = sum(lens[it[0]] for it in use)
    nbytes = 2 * len(heads) * keys * D * (1 if fp8 else 2)
    what = (f"sequences {[it[0] for it in use]} of the batch (KV lengths {[lens[it[0]] for it in use]}), "
            f"KV heads {heads[0]}-{heads[-1]} with their query groups: the CPU-seeded sample the GPU arm holds "
            f"at the same positions" + (", dequantize_kv_fp8 then attention" if fp8 else ""))
    return dt, nbytes, what, kind


def reference_line(args, base, world):
    dt, nbytes, what, kind = time_cpu(args.workload, args.steps, max(1, args.warmup), budget_s=150.0,
                                      batch=args.batch)
    val = nbytes / dt / 1e12
    line = dict(base)
    line.update({
        "impl": "reference", "value": val, "ms_per_step": dt * 1e3, "us_per_step": dt * 1e6,
        "scaling": "strong" if args.workload in ("headshard", "headshard_fp8", "seqshard") else "weak",
        "dtype": "f32 (bf16 inputs)",
        "config": static_config(args.workload, world, args.batch, args.page_size, args.gather, args.page_order),
        "cpu_baseline": {"value": val, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": what},
        "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    return line


# ----------------------------------------------------------------------------- GPU timing
def measure(wl: Workload, steps: int, warmup: int, preheat_s: float, sustain_s: float, dist, dev):
    """Time `steps` steps of a workload (one CUDA event pair around them, barrier and
    synchronize on both sides, maximum over ranks), then the same step over `sustain_s`."""
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def agree_max(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(n: int) -> float:
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        wl.run_steps(n)  # one event pair: an event after every launch would serialise them
        b.record()
        barrier()
        return agree_max(a.elapsed_time(b)) / n

    wl.run_steps(max(3, warmup))
    torch.cuda.synchronize(dev)
    est_ms = max(timed(5), 1e-3)
    # a short untimed run so that the SM clock has left its idle state; the count is agreed
    # between the ranks (steps with an exchange are collective)
    if preheat_s > 0:
        wl.run_steps(min(int(preheat_s * 1e3 / est_ms) + 1, 100000))
    ms = timed(steps)
    res = {"ms_per_step": ms}
    if sustain_s > 0:
        n = min(int(sustain_s * 1e3 / ms) + 1, 200000)
        sms = timed(n)
        res["sustained"] = {"us_per_step": sms * 1e3, "steps": n, "seconds": sms * n / 1e3}
    res["kernel_status"] = wl.status()
    return res


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, a device-to-device copy)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (an earlier measurement on this GPU type)"


def summarise(wl: Workload, res: dict, world: int, job_bytes: float, peak: float) -> dict:
    ms = res["ms_per_step"]
    out = {"config": wl.desc, "scaling": wl.scaling, "us_per_step": ms * 1e3,
           "tb_s": job_bytes / (ms * 1e-3) / 1e12,
           "frac": wl.bytes_per_step / (ms * 1e-3) / 1e9 / peak,
           "kernel_status": res["kernel_status"],
           "collective": wl.collective or "none",
           "algorithmic_bytes_per_step": int(job_bytes)}
    if "sustained" in res:
        s = res["sustained"]
        out["sustained"] = dict(s, tb_s=job_bytes / (s["us_per_step"] * 1e-6) / 1e12,
                                frac=wl.bytes_per_step / (s["us_per_step"] * 1e-6) / 1e9 / peak)
    return out


def api_call_cost(wl: Workload, calls: int = 200):
    """Microseconds per call of the drop-in entry gqa_decode_attention(q, k, v) in a plain
    Python loop (the reference's own benchmark method, benchmarks/bench_bandwidth.py:25-33 of
    the reference), on the K/V sets of the single-sequence workload."""
    G = wl.G
    q = wl.q[0]
    kv = [(k[0], v[0]) for k, v, _, _ in wl.sets]
    for i in range(20):
        G.gqa_decode_attention(q, *kv[i % len(kv)])
    torch.cuda.synchronize(wl.dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for i in range(calls):
        G.gqa_decode_attention(q, *kv[i % len(kv)])
    b.record()
    host_us = (time.perf_counter() - t0) / calls * 1e6
    torch.cuda.synchronize(wl.dev)
    return {"device_us_per_call": a.elapsed_time(b) / calls * 1e3, "host_us_per_call": host_us, "calls": calls}


def quantize_cost(dev, peak: float):
    """The kernels that produce the E4M3 caches (the step before the path): whole-cache
    quantisation of one K tensor of config 3's size through gqa_quantize_kv_fp8, and the
    per-token append of config 5's batch through gqa_quantize_append_fp8.  Algorithmic bytes of
    the former as its two kernels are written: the amax pass reads 2 B per element, the
    conversion pass reads 2 B and writes 1 B."""
    from gqa_decode_b200 import fp8_utils

    heads, s = 64, 32768  # 8 sequences x 8 KV heads of config 3
    sets = [torch.randn(heads, s, D, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(2)]
    for x in sets:
        fp8_utils._quantize_one_cuda(x)
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 10
    a.record()
    for i in range(n):
        fp8_utils._quantize_one_cuda(sets[i % 2])
    b.record()
    torch.cuda.synchronize(dev)
    us = a.elapsed_time(b) / n * 1e3
    nbytes = 5 * heads * s * D
    out = {"quantize_kv_fp8": {"us_per_call": us, "elements": heads * s * D, "algorithmic_bytes": nbytes,
                               "bytes_rule": "2 B read by the amax kernel + 2 B read and 1 B written by the conversion kernel, per element",
                               "gb_s": nbytes / (us * 1e-6) / 1e9, "frac": nbytes / (us * 1e-6) / 1e9 / peak,
                               "l2": "two input sets of 537 MB alternated"}}
    del sets
    bsz, hkv, smax = 64, 8, 8192
    kc = torch.zeros(bsz, hkv, smax, D, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    vc = torch.zeros_like(kc)
    kn = torch.randn(bsz, hkv, D, device=dev).to(torch.bfloat16)
    vn = torch.randn(bsz, hkv, D, device=dev).to(torch.bfloat16)
    sc = torch.full((bsz, hkv), 1.0 / 64, device=dev)
    pos = torch.full((bsz,), 100, dtype=torch.int32, device=dev)
    for _ in range(3):
        fp8_utils.append_kv_fp8(kn, vn, kc, vc, sc, sc, pos)
    torch.cuda.synchronize(dev)
    n = 50
    a.record()
    for i in range(n):
        fp8_utils.append_kv_fp8(kn, vn, kc, vc, sc, sc, pos)
    b.record()
    torch.cuda.synchronize(dev)
    out["append_kv_fp8"] = {"us_per_call": a.elapsed_time(b) / n * 1e3, "batch": bsz, "num_kv_heads": hkv,
                            "note": "one new token per sequence; launch-bound (64 KB moved), timed through the Python entry"}
    return out


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="headshard", choices=WORKLOADS)
    ap.add_argument("--page-size", type=int, default=64, help="paged workload: rows per page")
    ap.add_argument("--page-order", default="shuffled", choices=["shuffled", "sequential"],
                    help="paged workload: pool pages in random order, or each sequence's pages in a row")
    ap.add_argument("--batch", type=int, default=16, help="ragged / paged workloads: sequences per rank")
    ap.add_argument("--preheat-s", type=float, default=0.05,
                    help="seconds of untimed steps after the warm-up so the SM clock leaves its idle "
                         "state (0 for profiler runs)")
    ap.add_argument("--sustain-s", type=float, default=0.5,
                    help="length of the additional sustained timing of every workload (0: skip)")
    ap.add_argument("--gather", default="none", choices=["none", "fused", "nccl"],
                    help="headshard at N>1: leave outputs sharded, gather them inside the decode kernel, "
                         "or all-gather them with NCCL afterwards")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nvlink", "nccl"],
                    help="seqshard at N>1: exchange+merge inside the decode kernel, a separate peer-store "
                         "exchange+merge kernel, or NCCL all-gather + merge")
    ap.add_argument("--dependent-launch", type=int, default=1,
                    help="1: launch steps with programmatic stream serialization (a step's prologue "
                         "overlaps the previous step's tail)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="time the main workload only")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1 and args.impl != "reference":
        # convenience: re-launch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", "29511",
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))

    base = {"metric": "decode_attn_achieved_hbm_throughput", "unit": "TB/s", "n_gpus": max(world, args.gpus),
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "vs_baseline": None, "data": "synthetic"}

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(reference_line(args, base, max(world, args.gpus))), flush=True)
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

    _native.load()  # raises when the CUDA library is missing

    def build(name, **kw):
        return Workload(name, rank, world, dev, args.batch, kw.get("exchange", args.exchange),
                        kw.get("gather", args.gather), args.page_size, bool(args.dependent_launch),
                        args.page_order)

    def job_bytes_of(wl):
        nb = torch.tensor([float(wl.bytes_per_step)], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(nb, op=dist.ReduceOp.SUM)
        return nb.item()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    peak, peak_src = hbm_peak()
    wl = build(args.workload)
    sampler = ClockSampler(local_rank)
    sampler.start()
    res = measure(wl, args.steps, max(3, args.warmup), args.preheat_s, args.sustain_s, dist, dev)
    job_bytes = job_bytes_of(wl)

    # ---- end to end from pinned host buffers
    e2e = None
    if not args.no_e2e:
        k0, v0 = wl.sets[0][0], wl.sets[0][1]
        host = {"q": wl.q.cpu().pin_memory(), "k": k0.cpu().pin_memory(), "v": v0.cpu().pin_memory()}
        out_shape = wl.run_set0().shape
        out_host = torch.empty(out_shape, dtype=torch.bfloat16).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = out_host.numel() * out_host.element_size()
        n_e2e = max(3, min(args.steps, 10))

        def e2e_step():
            wl.q.copy_(host["q"], non_blocking=True)
            k0.copy_(host["k"], non_blocking=True)
            v0.copy_(host["v"], non_blocking=True)
            out = wl.run_set0()
            out_host.copy_(out, non_blocking=True)

        e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b) / n_e2e], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = (float(t.item()), h2d, d2h, n_e2e)
        del host, out_host
    clocks = sampler.stop()
    parity = wl.parity()
    main_entry = summarise(wl, res, world, job_bytes, peak)
    launches = args.steps * wl.launches_per_step
    bytes_per_step, fp8_main = wl.bytes_per_step, wl.fp8
    del wl
    torch.cuda.empty_cache()

    # ---- the other workloads, briefly, at the same N
    others = {}
    if not args.no_others:
        todo = [(n, {}) for n in WORKLOADS if n != args.workload]
        if world > 1:
            todo.append(("headshard", {"gather": "fused"}))
        for name, kw in todo:
            key = name + ("_gather_fused" if kw.get("gather") == "fused" else "")
            try:
                w2 = build(name, **kw)
                r2 = measure(w2, min(args.steps, 50), 5, args.preheat_s, args.sustain_s, dist, dev)
                entry = summarise(w2, r2, world, job_bytes_of(w2), peak)
                entry["parity"] = w2.parity()
                if name == "single":
                    entry["api"] = api_call_cost(w2)
                others[key] = entry
                del w2
            except Exception as e:  # a workload that cannot run is reported, not hidden
                others[key] = {"error": f"{type(e).__name__}: {e}"}
                if dist is not None:
                    raise
            torch.cuda.empty_cache()
        try:
            others["fp8_cache_producers"] = quantize_cost(dev, peak)
        except Exception as e:
            others["fp8_cache_producers"] = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()

    if rank == 0:
        ms_per_step = res["ms_per_step"]
        achieved = bytes_per_step / (ms_per_step * 1e-3) / 1e9
        ratio = DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE["e4m3" if fp8_main else "bf16"]
        line = dict(base)
        line.update({
            "value": job_bytes / (ms_per_step * 1e-3) / 1e12, "ms_per_step": ms_per_step,
            "us_per_step": ms_per_step * 1e3, "scaling": main_entry["scaling"],
            "dtype": "e4m3->bf16 mma, f32 accumulate" if fp8_main else "bf16 mma, f32 accumulate",
            "config": main_entry["config"],
            "algorithmic_bytes_per_step": int(job_bytes),
            "kernel_status": res["kernel_status"],
            "collective": main_entry["collective"],
            "timing": {"preheat_s": args.preheat_s, "dependent_launch": bool(args.dependent_launch),
                       "method": "one CUDA event pair around the K steps, barrier + synchronize on both sides, max over ranks"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_src,
                         "traffic": ratio * bytes_per_step, "traffic_source": "ncu dram bytes per algorithmic byte of this kernel, scaled to this launch",
                         "kernel": "gqa::decode_kernel", "avg_launch_ms": ms_per_step,
                         "frac_of_nominal_8TBps": achieved / 8000.0, "per": "GPU"},
            "parity": parity,
            "clocks": clocks,
            "gpu_launches": launches,
        })
        if "sustained" in main_entry:
            line["sustained"] = main_entry["sustained"]
        if e2e:
            line["e2e"] = {"value": job_bytes / (e2e[0] * 1e-3) / 1e12, "unit": "TB/s",
                           "ms_per_step": e2e[0], "steps": e2e[3],
                           "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2]}
        if others:
            line["others"] = others
        if world == 1 and not args.no_cpu:
            # the CPU baseline runs in a process of its own: the reference package and this
            # repository's drop-in package share the import name
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference",
                                "--workload", args.workload, "--steps", "2", "--warmup", "1",
                                "--batch", str(args.batch)], capture_output=True, text=True, timeout=900)
            try:
                ref = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
                line["cpu_baseline"] = dict(ref["cpu_baseline"], ms_per_sample=ref["ms_per_step"])
            except Exception:
                line["cpu_baseline"] = {"error": (r.stderr or r.stdout)[-300:]}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
