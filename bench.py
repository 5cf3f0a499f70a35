#!/usr/bin/env python
"""Benchmark of the int8 attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--gate on|off]

One JSON line on stdout (rank 0).  A step is one call of the public entry
``superl8_b200.attn_int8_fwd(q, k, v, causal=True)`` -- accuracy gate, Q/K quantisation
prologue and attention kernel -- on the 64-head causal S=8192 configuration ("cfg3":
B16 Hq64 Hkv8 S8192 D128, fp16 ~N(0,1), a seeded 1 % of Q and K channels x20).  With the
gate on (default, the reference's behaviour) those outlier channels demote the call to the
full-precision kernel; the same line also carries the pure int8 path (gate off), the
full-W8A8 route on a slice of the batch, the split-KV decode (cfg5, fp16 and int8 V), the
backward pair and the quantiser, each with its own roofline figures; ``e2e`` -- the same step
through ``attn_int8_fwd_host`` with Q, K, V and the output in pinned host memory, plus the
PCIe bandwidth measured on those buffers alone; ``strong`` -- ONE cfg3 batch / cfg5's 128
sequences split over the ranks; and ``shard_check`` -- a small batch computed sharded,
all-gathered over NCCL and compared bitwise with the unsharded result.
Every rank owns a full cfg3 batch (weak scaling over (batch, kv-head) units, no collective
in the timed region).  ``--impl reference`` times the CPU restatement of the reference's
path (oracle/) on the host cores instead.  ``--kernel-case NAME`` launches one kernel family
on a small case and prints nothing on stdout (for profilers).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "attn_int8_fwd_tops"
UNIT = "TOPS"
NOMINAL_INT8_TOPS = 4500.0
NOMINAL_HBM_GBS = 7700.0


def load_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs.

    nvidia-smi needs a few hundred ms before its first sample, so it is started before the warm-up
    (start() returns once the first sample is on disk) and every sample carries its timestamp;
    stop() keeps the samples that fall inside the wall-clock window of the timed region.  When
    that window is shorter than the sampling can resolve, the samples of warm-up + timed region
    (the same kernels, back to back) are used and the record says so."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            deadline = time.time() + 5.0
            while time.time() < deadline and os.path.getsize(self.path) == 0:
                time.sleep(0.02)
        except Exception:
            self.proc = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    @staticmethod
    def _epoch(stamp: str):
        import datetime
        try:
            return datetime.datetime.strptime(stamp, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 10:
                    continue
                try:
                    rows.append((self._epoch(f[0]), float(f[2]), float(f[3]), float(f[4]), f[6:10]))
                except ValueError:
                    continue
            os.unlink(self.path)
        except Exception:
            pass
        inside = [r for r in rows if r[0] is not None and self.t_begin is not None and self.t_end is not None
                  and self.t_begin <= r[0] <= self.t_end]
        window = "timed region"
        if len(inside) < 3:
            # the region is shorter than three sampling periods: use warm-up + timed region, and of
            # those only the samples taken under load (power well above idle)
            inside = [r for r in rows if r[3] > 400.0] or rows
            window = "warm-up + timed region (timed region shorter than three samples)"
        if inside:
            reasons = set()
            for r in inside:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            out.update(sm_mhz=statistics.median([r[1] for r in inside]), sm_max_mhz=max(r[2] for r in inside),
                       power_w=statistics.median([r[3] for r in inside]), reasons=sorted(reasons),
                       samples=len(inside), window=window)
        return out


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def timed(fn, steps: int, warmup: int, world: int, before=None, after=None):
    """W untimed steps, then exactly K steps between barrier + synchronize; CUDA events on the
    launching stream; MAX over ranks.  Returns ms per step."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if before is not None:
        before()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if after is not None:
        after()
    if world > 1:
        dist.barrier()
    from superl8_b200 import shard
    return shard.max_over_ranks(e0.elapsed_time(e1), device="cuda") / steps


def cpu_reference_sample(cfg, heads_groups: int, threads=None):
    """The reference's CPU path restated (oracle/): CPU quantiser + fp32 attention oracle on
    batch element 0, `heads_groups` KV groups (each with its Hq/Hkv query heads).
    Returns (seconds, ops of the sample)."""
    from oracle import oracle
    if threads:
        torch.set_num_threads(threads)
    g = cfg.Hq // cfg.Hkv
    q, k, v = oracle.make_qkv(3000, g * heads_groups, heads_groups, cfg.S, cfg.D)
    q, k, v = q[None], k[None], v[None]
    t0 = time.perf_counter()
    oracle.quantize_qk(q, k)
    for h in range(heads_groups):  # one KV group at a time bounds the fp32 score matrix
        oracle.attention_fp32(q[:, h * g:(h + 1) * g], k[:, h:h + 1], v[:, h:h + 1], causal=cfg.causal)
    dt = time.perf_counter() - t0
    ops = 4.0 * g * heads_groups * cfg.S * cfg.S * cfg.D * (0.5 if cfg.causal else 1.0)
    return dt, ops


def run_reference(args, cfg):
    rank, world, _ = dist_setup(args.gpus)
    if rank != 0:
        return
    # every host core this process may use (a launcher such as torchrun pins OMP_NUM_THREADS to 1)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    groups = 1
    for _ in range(args.warmup):
        cpu_reference_sample(cfg, groups)
    ts = []
    ops = 0.0
    for _ in range(args.steps):
        dt, ops = cpu_reference_sample(cfg, groups)
        ts.append(dt)
    sec = sum(ts) / len(ts)
    val = ops / sec / 1e12
    sample = f"batch element 0, {groups} KV group ({cfg.Hq // cfg.Hkv} query heads) of {cfg.name} per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args, max(1, args.gpus)),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def run_kernel_case(args):
    """Small, profiler-friendly cases (inputs larger than L2, about 1 GB on the device)."""
    import superl8_b200 as s8
    from superl8_b200 import _C, quant, workloads
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = args.warmup + args.steps
    if args.kernel_case in ("prefill_int8", "prefill_fp16", "prefill_w8a8", "quant_q", "quant_k", "quant_k_fused"):
        c = workloads.PrefillCfg("cfg3_b2", 2, 64, 8, 8192, 128, True)
        q, k, v = workloads.prefill_inputs(c, dev, outliers=False)
        if args.kernel_case == "prefill_fp16":
            for _ in range(n):
                _C.attn_fp16_fwd(q, k, v, True, None, -1, None)
        elif args.kernel_case == "quant_q":
            for _ in range(n):
                quant.quantize_q(q, 0.0884, want_gate=True)
        elif args.kernel_case == "quant_k":
            kk = torch.cat([k] * 8, dim=0)
            for _ in range(n):
                quant.smooth_quantize_k(kk, quant.k_mean(kk))
        elif args.kernel_case == "quant_k_fused":       # mean + smoothing + quantisation in one launch
            kk = torch.cat([k] * 8, dim=0)
            for _ in range(n):
                quant.k_prologue(kk)
        elif args.kernel_case == "prefill_w8a8":
            q_i8, q_scale, k_i8, k_scale, _ = s8.quantize_qk(q, k)
            qs, ks = q_scale.squeeze(-1).contiguous(), k_scale.squeeze(-1).contiguous()
            v_i8, v_scale = quant.quantize_v_perchannel(v)
            vs = v_scale.squeeze(-2).contiguous()
            for _ in range(n):
                _C.attn_w8a8_fwd(q_i8, qs, k_i8, ks, v_i8, vs, True, 0, True)
        else:
            q_i8, q_scale, k_i8, k_scale, _ = s8.quantize_qk(q, k)
            qs, ks = q_scale.squeeze(-1).contiguous(), k_scale.squeeze(-1).contiguous()
            for _ in range(n):
                _C.attn_int8_fwd(q_i8, qs, k_i8, ks, v, True, -1)
    elif args.kernel_case == "backward":
        g = torch.Generator(device="cpu").manual_seed(2002)
        bq, bk, bv, bdo = (torch.randn(2, h, 4096, 128, generator=g).half().to(dev) for h in (32, 8, 8, 32))
        bout, blse = _C.attn_fp16_fwd(bq, bk, bv, True, None, want_lse=True)
        for _ in range(n):
            s8.backward_cuda(bq, bk, bv, bout, blse, bdo, causal=True)
    else:
        dcfg = workloads.DecodeCfg(B=16)
        lens = workloads.decode_lengths(dcfg, 0, 16)
        dq, dk8, dks, dv, dlens = workloads.decode_inputs(dcfg, lens, dev)
        if args.kernel_case == "decode_kv8":
            dv8, dvs = quant.quantize_v_perchannel(dv)
            dvs = dvs.squeeze(-2).contiguous()
            for _ in range(n):
                s8.attn_decode_cached(dq, dk8, dks, dv8, dvs, context_lens=dlens)
        else:
            for _ in range(n):
                s8.attn_decode_int8_cache(dq, dk8, dks, dv, context_lens=dlens)
    torch.cuda.synchronize()
    print(f"kernel-case {args.kernel_case}: {n} launches, device status {_C.device_status()}", file=sys.stderr)


def shard_check(world, rank, dev):
    """One small batch computed sharded over the ranks, all-gathered over NCCL and compared BITWISE with
    the same batch computed whole on this GPU (outside every timed region): prefill through the public
    entry and ragged decode against a quantised cache.  Units are independent, so the two must be equal."""
    import torch.distributed as dist
    import superl8_b200 as s8
    from superl8_b200 import quant, shard, workloads
    c = workloads.PrefillCfg("cfg1_check", 8, 16, 4, 512, 128, True)
    q, k, v = workloads.prefill_inputs(c, dev, source="cpu")
    whole = s8.attn_int8_fwd(q, k, v, causal=True)
    b_rng, _ = shard.batch_range(c.B, c.Hkv, min(world, c.B), rank % min(world, c.B))
    sl = slice(b_rng.start, b_rng.stop)
    local = s8.attn_int8_fwd(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), causal=True)
    ok_p = torch.equal(shard.gather_batch(local), whole) if world <= c.B else True
    g = torch.Generator().manual_seed(5151)
    lens = torch.randint(300, 3000, (8,), generator=g, dtype=torch.int32)
    n_max = int(lens.max())
    dq = torch.randn(8, 16, 1, 128, generator=g).half().to(dev)
    kk = torch.randn(8, 4, n_max, 128, generator=g).half().to(dev)
    dv = torch.randn(8, 4, n_max, 128, generator=g).half().to(dev)
    ldev = lens.to(dev)
    k_i8, k_s, _ = quant.smooth_quantize_k(kk, quant.k_mean(kk, ldev))
    k_s = k_s.squeeze(-1).contiguous()
    whole_d = s8.attn_decode_int8_cache(dq, k_i8, k_s, dv, context_lens=ldev)
    local_d = s8.attn_decode_int8_cache(dq[sl].contiguous(), k_i8[sl].contiguous(), k_s[sl].contiguous(),
                                        dv[sl].contiguous(), context_lens=ldev[sl].contiguous())
    ok_d = torch.equal(shard.gather_batch(local_d), whole_d) if world <= 8 else True
    flag = torch.tensor([int(ok_p), int(ok_d)], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok_p, ok_d = bool(flag[0].item()), bool(flag[1].item())
    return {"prefill": "bitwise equal" if ok_p else "MISMATCH", "decode": "bitwise equal" if ok_d else "MISMATCH",
            "how": f"B8 Hq16 Hkv4 S512 D128 causal prefill and 8 ragged decode sequences: {min(world, 8)} shards, "
                   f"all_gather ({'nccl' if world > 1 else 'single rank'}), torch.equal with the unsharded result"}


def copy_bandwidth(hin, din, dout, hout, world, reps=3):
    """Pinned host <-> device copy rates of this step's buffers, per direction and both at once
    (GB/s per GPU, from the slowest rank's time): the floor under the end-to-end step."""
    import torch.distributed as dist
    from superl8_b200 import shard
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    res = {}
    for name, do_in, do_out in (("h2d_only", True, False), ("d2h_only", False, True), ("both", True, True)):
        best = None
        for _ in range(reps):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            if do_in:
                with torch.cuda.stream(s_in):
                    din.copy_(hin, non_blocking=True)
            if do_out:
                with torch.cuda.stream(s_out):
                    hout.copy_(dout, non_blocking=True)
            torch.cuda.synchronize()
            dt = shard.max_over_ranks(time.perf_counter() - t0, device="cuda")
            best = dt if best is None else min(best, dt)
        nbytes = (hin.numel() * hin.element_size() if do_in else 0) + (hout.numel() * hout.element_size() if do_out else 0)
        res[name] = {"gbs_per_gpu": nbytes / best / 1e9, "ms": best * 1e3}
    return res


def host_placement(local: int) -> dict:
    """Where this rank's host side sits relative to its GPU: the NUMA node of the GPU's PCIe slot, the
    NUMA nodes of the CPUs the process may run on (pinned buffers are first touched there) and how
    many CPUs that is.  Explains an end-to-end figure that does not scale with the GPUs: all ranks
    of a box share one host memory system."""
    out = {"cpus_allowed": len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()}
    try:
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        dom = torch.cuda.get_device_properties(local).pci_domain_id
        dev = torch.cuda.get_device_properties(local).pci_device_id
        path = Path(f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node")
        out["gpu_numa_node"] = int(path.read_text().strip()) if path.exists() else None
    except Exception:
        out["gpu_numa_node"] = None
    try:
        allowed = os.sched_getaffinity(0)
        nodes = []
        for node in sorted(Path("/sys/devices/system/node").glob("node[0-9]*")):
            cpus = set()
            for part in (node / "cpulist").read_text().strip().split(","):
                if part:
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            if cpus & allowed:
                nodes.append(int(node.name[4:]))
        out["cpu_numa_nodes"] = nodes
    except Exception:
        out["cpu_numa_nodes"] = None
    return out


def workload_config(cfg, args, world):
    return {"workload": f"{cfg.name}: attn_int8_fwd causal B{cfg.B} Hq{cfg.Hq} Hkv{cfg.Hkv} S{cfg.S} D{cfg.D} fp16 "
                        f"~N(0,1), 1% of Q/K channels x20, per GPU",
            "gate": args.gate, "per_gpu_batch": cfg.B, "global_batch": cfg.B * world,
            "sharding": f"{cfg.units} independent (batch, kv-head) units per GPU, no collective",
            "l2": "inputs (2.7 GB per step) larger than L2"}


_REAL_STDOUT = None


def quiet_stdout():
    """Libraries (NCCL's version banner, for one) write to fd 1; the contract is ONE JSON line
    there.  Everything but emit() goes to stderr from here on."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict):
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gate", default="on", choices=["on", "off"])
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--skip-extras", action="store_true", help="only the headline workload")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every GPU owns a full batch; strong: the batch's units are split across the GPUs")
    ap.add_argument("--kernel-case", default="", choices=["", "prefill_int8", "prefill_fp16", "prefill_w8a8", "quant_k_fused", "decode", "decode_kv8", "backward", "quant_q", "quant_k"],
                    help="launch ONE kernel family on a small case (for profilers): W warm-up + K launches, no JSON")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from superl8_b200 import workloads
    cfg = workloads.PREFILL[args.workload]
    if args.kernel_case:
        run_kernel_case(args)
        return
    if args.impl == "reference":
        run_reference(args, cfg)
        return

    import torch.distributed as dist
    import superl8_b200 as s8
    from superl8_b200 import _C, _lib, quant

    rank, world, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    gate = args.gate == "on"

    from superl8_b200 import shard
    total_ops = world * cfg.ops
    if args.scaling == "strong":   # this rank's slice of the ONE global batch
        b_rng, _h = shard.batch_range(cfg.B, 1, min(world, cfg.B), rank % min(world, cfg.B))
        total_ops = cfg.ops
        cfg = workloads.PrefillCfg(cfg.name, len(b_rng), cfg.Hq, cfg.Hkv, cfg.S, cfg.D, cfg.causal, cfg.outliers)
        q, k, v = workloads.prefill_inputs(cfg, dev, first_unit_batch=b_rng.start)
    else:
        q, k, v = workloads.prefill_inputs(cfg, dev, first_unit_batch=rank * cfg.B)
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    hout = torch.empty(q.shape, dtype=torch.float16).pin_memory()

    def step():
        return s8.attn_int8_fwd(q, k, v, causal=cfg.causal, internal_accuracy_gate=gate)

    def step_e2e():
        # the library's host-buffer entry point: pinned Q, K, V in, pinned output back, every step
        return s8.attn_int8_fwd_host(hq, hk, hv, hout, causal=cfg.causal, internal_accuracy_gate=gate)

    # measured tensor-pipe peaks (back-to-back tcgen05.mma on constant operands, burst clocks)
    probe_i8, probe_f16 = _C.tensor_peak(True, 8192), _C.tensor_peak(False, 8192)

    out = step()
    demoted = s8.ops.last_gate_decision
    dominant = "attn_fp16_fwd" if demoted else "attn_int8_fwd"
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = [0]

    def before():
        launches0[0] = _lib.launches
        sampler.mark_begin()
    ms = timed(step, args.steps, args.warmup, world, before=before, after=sampler.mark_end)
    gpu_launches = _lib.launches - launches0[0]
    clocks = sampler.stop() if rank == 0 else {}

    def kernel_ms_of(fn):
        """Average duration of the dominant kernel alone: K launches on the step's own inputs, each
        bracketed by CUDA events on the launching stream, right behind the timed region (same
        sustained clocks)."""
        for _ in range(2):
            fn()
        evs = []
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / len(evs)

    if demoted:
        kern_ms = kernel_ms_of(lambda: _C.attn_fp16_fwd(q, k, v, cfg.causal, None, -1, None))
    else:
        qi_, qs_, ki_, ks_, _m = s8.quantize_qk(q, k)
        qs_, ks_ = qs_.squeeze(-1).contiguous(), ks_.squeeze(-1).contiguous()
        kern_ms = kernel_ms_of(lambda: _C.attn_int8_fwd(qi_, qs_, ki_, ks_, v, cfg.causal, -1))
        del qi_, qs_, ki_, ks_
    status = _C.device_status()
    value = total_ops / (ms * 1e-3) / 1e12

    ms_e2e = timed(step_e2e, args.steps, args.warmup, world)
    e2e = {"value": total_ops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": sum(t.numel() * 2 for t in (hq, hk, hv)), "d2h_bytes_per_step": hout.numel() * 2,
           "entry": "sl8_attn_int8_fwd_host (chunks of (batch, kv-head) units on three streams, gate on the device)"}
    if not args.skip_extras:
        # what the PCIe link gives this step's buffers: Q alone in (2.1 GB), the output alone out, both at once
        e2e["copy_bandwidth"] = copy_bandwidth(hq, q, out, hout, world)
        e2e["host"] = host_placement(local)

    # DRAM traffic per launch from the ncu captures summarised under profiles/ (a B = 2 slice of
    # cfg3 for prefill, 1 M rows for the quantiser, 16 sequences for decode), scaled to this launch
    # by the units processed (traffic grows in proportion to them).
    NCU_TRAFFIC = {"attn_int8_fwd": 406.1e6 / 2, "attn_fp16_fwd": 562.8e6 / 2}   # bytes per batch element of cfg3

    def tensor_roofline(kernel_ms, note, key):
        ach = cfg.ops / (kernel_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"]   # the kernel runs inside a seconds-long, power-capped loop
        return {"bound": "tensor", "kernel": note, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak, "peak_source": peaks["source"] + " bf16 dense (sustained)",
                "frac_of_burst_bf16": ach / peaks["bf16_tflops"], "frac_of_nominal_int8": ach / NOMINAL_INT8_TOPS,
                "frac_of_probed_int8": ach / probe_i8, "frac_of_probed_f16": ach / probe_f16,
                "frac_of_probed_mixed_ceiling": ach / (1.0 / (0.5 / probe_i8 + 0.5 / probe_f16)),
                # one exponential per logit on a unit that delivers 16 per clock and SM: 4 * D operations ride on
                # each, so softmax without exponentials elsewhere cannot pass 16 * 4 * D * SMs * clock
                "exp_unit_ceiling": {"at_max_clock": 16 * 4 * cfg.D * 148 * (clocks.get("sm_max_mhz") or 1965.0) * 1e6 / 1e12,
                                     "at_sampled_clock": 16 * 4 * cfg.D * 148 * (clocks.get("sm_mhz") or 1965.0) * 1e6 / 1e12,
                                     "unit": "T(FL)OP/s",
                                     "frac_at_sampled_clock": ach / (16 * 4 * cfg.D * 148 * (clocks.get("sm_mhz") or 1965.0) * 1e6 / 1e12)},
                "traffic": NCU_TRAFFIC[key] * cfg.B, "ms_per_launch": kernel_ms}

    roofline = tensor_roofline(kern_ms, dominant + (" (gate demoted the call)" if demoted else ""), dominant)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f16" if demoted else "s8", "data": "synthetic", "config": workload_config(cfg, args, world),
        "gate_demoted": bool(demoted), "device_status": status, "e2e": e2e, "gpu_launches": gpu_launches,
        "clocks": clocks, "roofline": roofline,
        "tensor_peak_probe": {"int8_tops": probe_i8, "f16_tflops": probe_f16,
                              "how": "sl8_tensor_peak_probe: 148 blocks x 8192 x 4 tcgen05.mma M128 N256, constant operands"},
    }

    if not args.skip_extras:
        # ---- pure int8 path on the same inputs (gate off) ----
        ms8 = timed(lambda: s8.attn_int8_fwd(q, k, v, causal=cfg.causal, internal_accuracy_gate=False),
                    args.steps, args.warmup, world)
        qi_, qs_, ki_, ks_, _m = s8.quantize_qk(q, k)
        qs_, ks_ = qs_.squeeze(-1).contiguous(), ks_.squeeze(-1).contiguous()
        k8 = kernel_ms_of(lambda: _C.attn_int8_fwd(qi_, qs_, ki_, ks_, v, cfg.causal, -1))
        del qi_, qs_, ki_, ks_
        r8 = tensor_roofline(k8, "attn_int8_fwd (tcgen05 kind::i8 QK, kind::f16 PV)", "attn_int8_fwd")
        r8["frac_of_mixed_ceiling_nominal"] = r8["achieved"] / (NOMINAL_INT8_TOPS * 2.0 / 3.0)
        line["int8_path"] = {"value": total_ops / (ms8 * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms8,
                             "gate": "off", "roofline": r8}
        del out
        # ---- full W8A8 (P on the int8 grid, int8 V) on a two-element slice of the batch ----
        wq, wk, wv = (t[:2] for t in (q, k, v))
        wqi, wqs, wki, wks, _m = s8.quantize_qk(wq, wk)
        wqs, wks = wqs.squeeze(-1).contiguous(), wks.squeeze(-1).contiguous()
        wvi, wvs = quant.quantize_v_perchannel(wv)
        wvs = wvs.squeeze(-2).contiguous()
        w_ops = cfg.ops * wq.shape[0] / cfg.B
        ms_w = timed(lambda: _C.attn_w8a8_fwd(wqi, wqs, wki, wks, wvi, wvs, cfg.causal, 0, True), args.steps, args.warmup, world)
        ms_wm = timed(lambda: _C.attn_w8a8_fwd(wqi, wqs, wki, wks, wvi, wvs, cfg.causal, 0, True, backend=_lib.SL8_BACKEND_MMA),
                      1, 1, world)
        line["w8a8"] = {"metric": "attn_w8a8_fwd_tops", "value": world * w_ops / (ms_w * 1e-3) / 1e12, "unit": UNIT,
                        "ms_per_step": ms_w,
                        "config": {"workload": f"first {wq.shape[0]} batch elements of {cfg.name}, per GPU; int8 Q, K, V, "
                                               "P re-quantised per row and 32-key half"},
                        "kernel": "fwd_tc_kernel W8 (tcgen05 kind::i8 QK; P snapped to the int8 grid, kind::f16 PV on the codes) "
                                  "+ v_codes_kernel",
                        "mma_sync_kernel": {"value": world * w_ops / (ms_wm * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_wm},
                        "roofline": {"bound": "tensor", "achieved": w_ops / (ms_w * 1e-3) / 1e12,
                                     "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                                     "frac": w_ops / (ms_w * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                                     "peak_source": peaks["source"] + " bf16 dense (sustained)", "traffic": None}}
        del wq, wk, wv, wqi, wqs, wki, wks, wvi, wvs
        # ---- the experiment the configurations describe: ONE global batch, sharded over the GPUs ----
        b_rng, _h = shard.batch_range(cfg.B, cfg.Hkv, min(world, cfg.B), rank % min(world, cfg.B))
        qs_, ks_, vs_ = (t[b_rng.start:b_rng.stop] for t in (q, k, v))
        ms_s = timed(lambda: s8.attn_int8_fwd(qs_, ks_, vs_, causal=cfg.causal, internal_accuracy_gate=gate),
                     args.steps, args.warmup, world)
        v_s = cfg.ops / (ms_s * 1e-3) / 1e12
        line["strong"] = {"prefill": {"value": v_s, "unit": UNIT, "ms_per_step": ms_s, "global_batch": cfg.B,
                                      "per_gpu_batch": len(b_rng), "split": "shard.batch_range: whole batch elements per rank",
                                      "efficiency_vs_one_gpu": v_s / value if world > 1 else 1.0,
                                      "efficiency_note": "strong value / weak value of this run (weak value = N x one GPU's "
                                                         "throughput on the full batch)"}}
        del qs_, ks_, vs_
        # ---- quantiser (Q prologue with the gate statistic, on cfg3's Q) ----
        qbytes = q.numel() * 3 + (q.numel() // cfg.D) * 4
        msq = timed(lambda: quant.quantize_q(q, 0.0884, want_gate=True), args.steps, args.warmup, world)
        gq = world * qbytes / (msq * 1e-3) / 1e9
        line["quant"] = {"value": gq, "unit": "GB/s", "ms_per_step": msq, "what": "Q prologue (quantise + fold + gate) on cfg3 Q",
                         "roofline": {"bound": "hbm", "achieved": gq / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": gq / world / peaks["hbm_gbs"], "frac_of_nominal": gq / world / NOMINAL_HBM_GBS,
                                      "peak_source": peaks["source"] + " copy bandwidth",
                                      "traffic": 378.2e6 / 1048576 * (q.numel() // cfg.D)}}
        # ---- decode (cfg5): every rank owns 128 sequences ----
        del q, k, v
        torch.cuda.empty_cache()
        dcfg = workloads.DecodeCfg()
        lens = workloads.decode_lengths(dcfg, first_seq=0, count=dcfg.B)
        dq, dk8, dks, dv, dlens = workloads.decode_inputs(dcfg, lens, dev)
        dbytes = workloads.decode_bytes(lens, dcfg.Hkv, dcfg.D)
        launches1 = _lib.launches
        msd = timed(lambda: s8.attn_decode_int8_cache(dq, dk8, dks, dv, context_lens=dlens), max(args.steps, 10),
                    args.warmup, world)
        per_step = (_lib.launches - launches1) // (max(args.steps, 10) + args.warmup)
        gd = world * dbytes / (msd * 1e-3) / 1e9
        line["decode"] = {"metric": "int8_kv_decode_hbm_gbs", "value": gd, "unit": "GB/s", "ms_per_step": msd,
                          "gpu_launches_per_step": per_step,
                          "config": {"workload": "cfg5: B128 Hq64 Hkv8 D128, context uniform in [1024, 32768], int8 K + "
                                                 "fp32 per-token scales, fp16 V, per GPU",
                                     "l2": "K/V caches (13 GB) larger than L2"},
                          "roofline": {"bound": "hbm", "achieved": gd / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": gd / world / peaks["hbm_gbs"], "frac_of_nominal": gd / world / NOMINAL_HBM_GBS,
                                       "peak_source": peaks["source"] + " copy bandwidth",
                                       "traffic": 794.5e6 / 775.8e6 * dbytes},
                          "device_status": _C.device_status()}
        # strong decode: the 128 sequences of the ONE global batch, longest-first balanced over the ranks
        owned = shard.balance_by_length(lens.tolist(), world)[rank]
        if world > 1:
            idx = torch.tensor(owned, device=dev)
            sq, sk8, sks, sv, sl_ = (t.index_select(0, idx).contiguous() for t in (dq, dk8, dks, dv, dlens))
        else:
            sq, sk8, sks, sv, sl_ = dq, dk8, dks, dv, dlens
        msds = timed(lambda: s8.attn_decode_int8_cache(sq, sk8, sks, sv, context_lens=sl_), max(args.steps, 10),
                     args.warmup, world)
        gds = dbytes / (msds * 1e-3) / 1e9
        line["strong"]["decode"] = {"value": gds, "unit": "GB/s", "ms_per_step": msds, "global_sequences": dcfg.B,
                                    "per_gpu_sequences": len(owned), "split": "shard.balance_by_length (longest first)",
                                    "efficiency_vs_one_gpu": gds / gd if world > 1 else 1.0}
        del sq, sk8, sks, sv, sl_
        # ---- the same decode against an int8 V cache (per-channel scales): D + 4 + D bytes per key ----
        dv8, dvs = quant.quantize_v_perchannel(dv)
        dvs = dvs.squeeze(-2).contiguous()
        del dv
        d8bytes = sum(int(n) for n in lens) * dcfg.Hkv * (2 * dcfg.D + 4)
        msd8 = timed(lambda: s8.attn_decode_cached(dq, dk8, dks, dv8, dvs, context_lens=dlens), max(args.steps, 10),
                     args.warmup, world)
        gd8 = world * d8bytes / (msd8 * 1e-3) / 1e9
        line["decode_kv8"] = {"metric": "int8_kv_decode_hbm_gbs", "value": gd8, "unit": "GB/s", "ms_per_step": msd8,
                              "config": {"workload": "cfg5 with an int8 V cache (one fp32 scale per channel): "
                                                     "2D + 4 bytes per key and KV head"},
                              "roofline": {"bound": "hbm", "achieved": gd8 / world, "peak": peaks["hbm_gbs"],
                                           "unit": "GB/s", "frac": gd8 / world / peaks["hbm_gbs"],
                                           "frac_of_nominal": gd8 / world / NOMINAL_HBM_GBS,
                                           "peak_source": peaks["source"] + " copy bandwidth",
                                           # ncu, 16 sequences: 534.6 MB moved for 519.9 MB algorithmic
                                           "traffic": 534.6e6 / 519.9e6 * d8bytes},
                              "speedup_vs_fp16_v": msd / msd8}
        del dq, dk8, dks, dv8, dvs
        # ---- backward (dQ pass + dK/dV pass) on a cfg2-shaped training step per rank ----
        bB, bHq, bHkv, bS, bD = 2, 32, 8, 4096, 128
        gb = torch.Generator(device="cpu").manual_seed(2002 + rank)
        bq, bk, bv, bdo = (torch.randn(bB, h, bS, bD, generator=gb).half().to(dev) for h in (bHq, bHkv, bHkv, bHq))
        bout, blse = _C.attn_fp16_fwd(bq, bk, bv, True, None, want_lse=True)
        msb = timed(lambda: s8.backward_cuda(bq, bk, bv, bout, blse, bdo, causal=True), args.steps, args.warmup, world)
        bflops = 10.0 * bB * bHq * bS * bS * bD * 0.5      # five contractions, causal half
        tb = world * bflops / (msb * 1e-3) / 1e12
        line["backward"] = {"metric": "attn_bwd_tflops", "value": tb, "unit": "TFLOP/s", "ms_per_step": msb,
                            "config": {"workload": f"B{bB} Hq{bHq} Hkv{bHkv} S{bS} D{bD} causal fp16, per GPU",
                                       "flops": "10*B*Hq*S^2*D/2 (dV, dP, S, dQ, dK)"},
                            "roofline": {"bound": "tensor", "achieved": tb / world, "peak": peaks["bf16_tflops"],
                                         "unit": "TFLOP/s", "frac": tb / world / peaks["bf16_tflops"],
                                         "peak_source": peaks["source"] + " bf16 dense (burst)",
                                         # ncu on this shape: dQ pass 213.6 MB + dK/dV pass 328.2 MB
                                         "traffic": 541.8e6,
                                         "kernels": "bwd_tc_kernel dQ pass + dK/dV pass (tcgen05.mma kind::f16, TMA tiles, "
                                                    "accumulators in tensor memory)"}}
        del bq, bk, bv, bdo, bout, blse

    line["shard_check"] = shard_check(world, rank, dev)
    if rank == 0 and world == 1:
        try:
            torch.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
            sec, ops = cpu_reference_sample(cfg, 16)
            line["cpu_baseline"] = {"value": ops / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"16 KV groups (128 query heads = 2 batch elements) of {cfg.name}: CPU quantiser + "
                                              f"fp32 attention oracle, {sec:.1f} s"}
        except Exception as e:  # the CPU leg must never take the GPU numbers down with it
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"failed: {e!r}"}
    if rank == 0:
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
