#!/usr/bin/env python
"""Benchmark of the fused relative-position-bias attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass of the hot path over one batch of synthetic
input: fused-bias attention at the 8k-token point (T5-base heads: batch 2,
12 heads x 64, 8192 queries x 8192 keys, bf16, bidirectional buckets 32/128,
no 1/sqrt(d) scale).  With N > 1 (launched by torchrun, one rank per GPU) every
rank runs its own batch shard -- attention is independent per batch row, so
there is no data-path collective -- and the value is the whole-job aggregate
(weak scaling).  Rank 0 prints ONE JSON line.

`--impl reference` times the reference's own CPU `basic` path (the oracle port:
bucket grid + bias lookup + einsum/softmax/einsum, all host threads) on a
bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name="fused-bias attention fwd, T5-base heads @8k", B=2, H=12, L=8192, D=64,
                num_buckets=32, max_distance=128)
L2_BYTES = 126 * 1024 * 1024
# DRAM traffic (read + write) of one launch of the forward kernel on the workload above,
# from an ncu capture of that launch (dram__bytes_read.sum + dram__bytes_write.sum).
NCU_DRAM_BYTES_PER_LAUNCH = 75.6e6 + 10.7e6


def _bind_to_gpu_numa_node(index):
    """Run this process on the CPUs of the NUMA node its GPU hangs off, before any pinned host buffer is
    allocated: the end-to-end leg copies 100 MB per step over PCIe, and with several ranks on one host the
    copies of all of them otherwise share whichever node the buffers happened to land on.  Returns the
    node, or None when the machine does not say (then nothing is changed)."""
    try:
        pr = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        node = int(open("/sys/bus/pci/devices/" + bdf + "/numa_node").read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)          # never widen what the launcher allowed
        if not cpus:
            return None
        _bind_to_gpu_numa_node.before = os.sched_getaffinity(0)
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def flops_per_step(w):
    return 4.0 * w["B"] * w["H"] * w["L"] * w["L"] * w["D"]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), hbm=float(p["hbm_gbs"]), source="measured (burst)")
    return dict(tflops=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the GPU is under load."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.06)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                clk, mx, util = float(parts[1]), float(parts[2]), float(parts[4])
            except ValueError:
                continue
            smax = mx
            if util >= 50:
                sm.append(clk)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[6:10]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=smax,
                    reasons=sorted(reasons), samples_under_load=len(sm))


def _reference_functions():
    """The reference's own `basic` pieces (T5Attention._relative_position_bucket,
    naive_torch_attention_with_bias) when its source tree can be imported on this machine
    (an install under baseline/_ref, a checkout named by TURBOT5_REFERENCE_SRC, or a `reference`
    checkout beside this repository), else None.  The three symbols the installed `transformers` no
    longer has are stubbed first; none is on this path."""
    import types
    roots = [os.path.join(ROOT, "baseline", "_ref"), os.environ.get("TURBOT5_REFERENCE_SRC", ""),
             os.path.join(os.path.dirname(ROOT), "reference", "src")]
    for root in roots:
        if not root or not os.path.isdir(os.path.join(root, "turbot5")):
            continue
        try:
            import transformers.pytorch_utils as pu
            if not hasattr(pu, "find_pruneable_heads_and_indices"):
                pu.find_pruneable_heads_and_indices = lambda *a, **k: None
            m = types.ModuleType("transformers.utils.model_parallel_utils")
            m.assert_device_map = lambda *a, **k: None
            m.get_device_map = lambda *a, **k: {}
            sys.modules.setdefault("transformers.utils.model_parallel_utils", m)
            o = types.ModuleType("transformers.onnx")
            o.OnnxSeq2SeqConfigWithPast = type("OnnxSeq2SeqConfigWithPast", (), {})
            sys.modules.setdefault("transformers.onnx", o)
            sys.path.insert(0, root)
            from turbot5.model.attentions import T5Attention
            from turbot5.ops.naive_attention import naive_torch_attention_with_bias
            return T5Attention._relative_position_bucket, naive_torch_attention_with_bias
        except Exception:
            if sys.path and sys.path[0] == root:
                sys.path.pop(0)
    return None


def cpu_attention_sample(w, pairs, threads, ref=None):
    """The reference's `basic` path on `pairs` (batch, head) pairs of the workload, all query rows,
    float32 arithmetic on bf16 values; returns seconds.  With `ref` (the reference's own bucket and
    attention functions) those run, slab by slab of 1024 query rows so that the L x L tensors never
    exist whole; otherwise the oracle port of the same steps."""
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    L, D = w["L"], w["D"]
    q = torch.randn((1, pairs, L, D), generator=g).bfloat16()
    k = torch.randn((1, pairs, L, D), generator=g).bfloat16()
    v = torch.randn((1, pairs, L, D), generator=g).bfloat16()
    table = (torch.randn((w["num_buckets"], pairs), generator=g) * 0.1).bfloat16()
    t0 = time.perf_counter()
    if ref is None:
        from oracle import t5_oracle as orc
        orc.attention_basic(q, k, v, table, causal=False, num_buckets=w["num_buckets"],
                            max_distance=w["max_distance"], slab=1024)
    else:
        bucket_fn, attn_fn = ref
        kf, vf, tf = k.float(), v.float(), table.float()
        mem = torch.arange(L)[None, :]
        for r0 in range(0, L, 1024):
            ctx = torch.arange(r0, min(r0 + 1024, L))[:, None]
            bucket = bucket_fn(mem - ctx, bidirectional=True, num_buckets=w["num_buckets"],
                               max_distance=w["max_distance"])
            bias = tf[bucket].permute(2, 0, 1).unsqueeze(0)
            attn_fn(q[:, :, r0:r0 + 1024].float(), kf, vf, bias)
    return time.perf_counter() - t0


REF_STEPS_CAP = 3       # a step of the CPU arm takes about ten seconds


def run_reference(args, rank, world):
    """Reference arm: the CPU `basic` path over the whole workload (all batch x head pairs, every
    host thread), rank 0 only.  --steps / --warmup are honoured up to REF_STEPS_CAP / 1."""
    if rank != 0:
        return
    w = WORKLOAD
    cores = os.cpu_count() or 1
    pairs = w["B"] * w["H"]
    ref = _reference_functions()
    steps, warmup = max(1, min(args.steps, REF_STEPS_CAP)), min(args.warmup, 1)
    for _ in range(warmup):
        cpu_attention_sample(w, pairs, cores, ref)
    times = [cpu_attention_sample(w, pairs, cores, ref) for _ in range(steps)]
    sec = sum(times) / len(times)
    val = flops_per_step(w) / sec / 1e12
    kind = "reference" if ref is not None else "port"
    sample = (f"all {pairs} (batch, head) pairs of the workload per step, float32 arithmetic on bf16 values, "
              f"{'the reference tree imported on this machine' if ref else 'oracle port (no reference tree on this machine)'}; "
              f"steps capped at {REF_STEPS_CAP}, warm-up at 1")
    line = {
        "impl": "reference", "metric": "fused_bias_attention_fwd_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": w["name"], "B": w["B"], "H": w["H"], "M": w["L"],
                                        "N": w["L"], "D": w["D"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


_JSON_FD = None


def _keep_stdout_for_json():
    """Library banners (NCCL prints its version on stdout when the first communicator is made) must not
    land beside the one JSON line: file descriptor 1 is pointed at stderr for the run and the line is
    written to the saved descriptor."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(line):
    text = json.dumps(line) + "\n"
    if _JSON_FD is not None:
        sys.stdout.flush()
        os.write(_JSON_FD, text.encode())
    else:
        print(text, end="", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000, help="timed steps (default: about 0.6 s of kernel time)")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary kernel measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--train", action="store_true",
                    help="time forward + backward of the same workload (the training step of the attention core) "
                         "instead of the forward: a second workload, used for the backward kernels' profile")
    ap.add_argument("--kernel", default="auto", choices=["auto", "tcgen05", "tcgen05_2tile", "tcgen05_polyexp", "simt"],
                    help="kernel of the attention step (default: the library's choice); the others exist for "
                         "comparisons and profiles")
    ap.add_argument("--workload", default="attention", choices=["attention", "encoder", "token_kernels"],
                    help="attention: the headline step.  encoder / token_kernels: second workloads on one GPU, used "
                         "for profiles -- a fused T5-base encoder pass over 2 x 8192 tokens per step, or one launch "
                         "each of the token-wise kernels (RMSNorm, residual add + RMSNorm, gated GELU, merge) per step")
    ap.add_argument("--head-dim", type=int, default=64, choices=[64, 128],
                    help="64: the headline workload; 128: the same workload at the T5-3B/11B head size "
                         "(a second tile geometry of the kernel; used for its profile)")
    args = ap.parse_args()
    if args.impl != "reference":
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    import turbot5_b200 as t5b
    from turbot5_b200 import _native as nat
    nat.lib()   # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: turbot5_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = _bind_to_gpu_numa_node(local)
    if world > 1:
        _keep_stdout_for_json()
        # The collectives of the sequence-parallel leg run on a high-priority stream: their few blocks are then
        # scheduled ahead of the attention blocks still waiting for an SM, so the gather really starts while the
        # attention over the local keys runs.
        opts = None
        if os.environ.get("T5B_BENCH_NCCL_PRIORITY", "1") != "0":
            from torch.distributed import ProcessGroupNCCL
            opts = ProcessGroupNCCL.Options()
            opts.is_high_priority_stream = True
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)

    if args.workload != "attention":
        side_workload(args, t5b, dev)
        return

    w = dict(WORKLOAD)
    if args.kernel != "auto":
        w["name"] += f" (kernel={args.kernel})"
    if args.head_dim != w["D"]:
        w.update(D=args.head_dim, name=f"fused-bias attention fwd, 12 heads of dim {args.head_dim} @8k")
    B, H, L, D = w["B"], w["H"], w["L"], w["D"]
    dt = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    set_bytes = 3 * B * H * L * D * 2
    n_sets = max(2, -(-int(1.5 * L2_BYTES) // set_bytes))        # rotating inputs exceed the L2

    def make_set():
        # (B,H,L,D) views of (B,L,H,D) buffers: the layout the attention module produces
        return [torch.randn((B, L, H, D), generator=g, device=dev, dtype=torch.float32).to(dt).transpose(1, 2)
                for _ in range(3)]
    sets = [make_set() for _ in range(n_sets)]
    table = (torch.randn((w["num_buckets"], H), generator=g, device=dev) * 0.1).to(dt)

    if args.train:
        w["name"] += ", forward + backward"
        for st_ in sets:
            for t_ in st_:
                t_.requires_grad_(True)
        table.requires_grad_(True)
        dout = torch.randn((B, H, L, D), generator=g, device=dev, dtype=torch.float32).to(dt)

    def step(i):
        q, k, v = sets[i % n_sets]
        o_ = t5b.flash_attention_with_fusing_bias(q, k, v, table, causal=False, sm_scale=1.0,
                                                  NUM_BUCKETS=w["num_buckets"], MAX_DISTANCE=w["max_distance"],
                                                  kernel=args.kernel)
        if args.train:
            torch.autograd.grad(o_, (q, k, v, table), dout)     # gradients only: no accumulation kernels in the step
        return o_

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    t5b.check_device_status(dev)
    ms_step = ms_total / args.steps
    # forward: 2 matrix products; training step: + the 5 a backward needs (2.5 x forward)
    fl = flops_per_step(w) * (3.5 if args.train else 1.0)
    value = world * fl / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers (pinned): every step copies its
    # q/k/v from the host, runs the attention call and copies the result back.  The copies run
    # on their own streams with two buffer slots, so that the upload of step i+1 and the
    # download of step i-1 overlap the kernel of step i (as a serving loop would do it).
    e2e_steps = max(3, min(args.steps, 20))
    # q, k and v of a step sit in ONE pinned host buffer and travel with one copy (three copies of a third each
    # reached 50 GB/s on this host)
    host_sets = [torch.stack([t_.detach().contiguous().cpu() for t_ in sets[i % n_sets]]).pin_memory() for i in range(2)]
    host_out = [torch.empty((B, H, L, D), dtype=dt).pin_memory() for _ in range(2)]
    dev_in = [torch.empty((3, B, H, L, D), dtype=dt, device=dev) for _ in range(2)]
    main = torch.cuda.current_stream(dev)
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        s_ = i % 2
        with torch.cuda.stream(up):
            up.wait_event(ev_done[s_])            # the kernel that last read this slot has finished
            dev_in[s_].copy_(host_sets[s_], non_blocking=True)
            ev_in[s_].record(up)
        main.wait_event(ev_in[s_])
        o = t5b.flash_attention_with_fusing_bias(dev_in[s_][0], dev_in[s_][1], dev_in[s_][2], table.detach(), causal=False,
                                                 sm_scale=1.0, NUM_BUCKETS=w["num_buckets"],
                                                 MAX_DISTANCE=w["max_distance"])
        ev_done[s_].record(main)
        with torch.cuda.stream(down):
            down.wait_event(ev_done[s_])
            host_out[s_].copy_(o, non_blocking=True)
            o.record_stream(down)
            ev_out[s_].record(down)

    def e2e_drain():
        for e_ in ev_out:
            main.wait_event(e_)
    for i in range(4):
        e2e_step(i)
    e2e_drain()
    barrier()
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_drain()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    e2e_val = world * fl / (e2e_ms * 1e-3) / 1e12

    secondary = None
    sp_line = None
    cfg2_line = None
    if not args.no_secondary:
        sp_line = sequence_parallel_measurement(t5b, dev, rank, world, dist)
        cfg2_line = config2_measurement(t5b, dev, rank, world, dist)
    if not args.no_secondary and rank == 0:
        secondary = secondary_measurements(t5b, dev)
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        peaks = measured_peaks()
        achieved = fl / (ms_step * 1e-3) / 1e12
        line = {
            "metric": "fused_bias_attention_fwd_bwd_tflops" if args.train else "fused_bias_attention_fwd_tflops",
            "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "B_per_gpu": B, "H": H, "M": L, "N": L, "D": D,
                       "num_buckets": w["num_buckets"], "max_distance": w["max_distance"], "causal": False,
                       "sm_scale": 1.0, "layout": "BHLD views of BLHD buffers", "parallelism": f"batch-sharded x{world}",
                       "l2": f"inputs rotate over {n_sets} sets ({n_sets * set_bytes / 2**20:.0f} MiB > 126 MiB L2)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops"],
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH if (D == WORKLOAD["D"] and not args.train) else None,
                         "traffic_source": "ncu capture of one launch of this kernel on this workload "
                                           "(profiles/attn_fwd_sm100_8k.md); algorithmic Q+K+V+O = "
                                           f"{4 * B * H * L * D * 2 / 1e6:.1f} MB",
                         "peak_source": peaks["source"],
                         "kernel": "attn_fwd_kernel + attn_bwd_dq_kernel + attn_bwd_dkv_wide_kernel" if args.train
                                   else "attn_fwd_kernel<bf16>"},
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": set_bytes,
                    "d2h_bytes_per_step": B * H * L * D * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "host_numa_node_rank0": numa},
            "gpu_launches": args.steps * (4 if args.train else 1),
            "clocks": clocks,
        }
        if clocks and clocks.get("sm_mhz"):
            # clock-independent form of the step time: SM cycles (in millions) per step at the median clock seen
            line["mcycles_per_step"] = ms_step * clocks["sm_mhz"] / 1e3
            line["timed_region_s"] = ms_total / 1e3
        if world == 1 and not args.no_cpu_baseline:
            before = getattr(_bind_to_gpu_numa_node, "before", None)
            if before:                                  # the CPU baseline takes every core the launcher allowed
                os.sched_setaffinity(0, before)
            cores = os.cpu_count() or 1
            pairs = B * H
            ref = _reference_functions()
            sec = cpu_attention_sample(w, pairs, cores, ref)
            line["cpu_baseline"] = {
                "value": flops_per_step(w) / sec / 1e12, "unit": "TFLOP/s", "cores": cores,
                "kind": "reference" if ref is not None else "port",
                "sample": f"all {pairs} (batch, head) pairs, all {L} rows, one pass: {sec:.1f} s of CPU work"}
        if secondary:
            line["secondary"] = secondary
        if sp_line:
            line["sequence_parallel"] = sp_line
        if cfg2_line:
            line["t5_base_encoder_decoder_16x1024"] = cfg2_line
        _emit(line)
    if world > 1:
        dist.destroy_process_group()


def token_kernel_measurements(t5b, dev, iters=30):
    """HBM-bound token-wise kernels at T5-base sizes (100 000 tokens: every operand larger than L2 or
    rotated out by the others): algorithmic bytes / device time."""
    from turbot5_b200.attention import merge_attention_partials
    peaks = measured_peaks()
    dt = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(11)
    rows, d, f = 100000, 768, 2048
    out = {}
    x = torch.randn((rows, d), generator=g, device=dev).to(dt)
    br = torch.randn((rows, d), generator=g, device=dev).to(dt)
    wgt = torch.rand((d,), generator=g, device=dev).to(dt)
    steps = {}
    steps["rmsnorm_100000x768_bf16"] = (lambda: t5b.rms_layer_norm(x, wgt, 1e-6), 2 * rows * d * 2 + d * 2)
    steps["add_rmsnorm_100000x768_bf16"] = (lambda: t5b.add_rms_layer_norm(x, br, wgt, 1e-6), 4 * rows * d * 2 + d * 2)
    h = torch.randn((rows, 2 * f), generator=g, device=dev).to(dt)
    steps["gated_gelu_100000x2048_bf16"] = (lambda: t5b.gated_gelu(h), 3 * rows * f * 2)
    M = 12500
    # (two sets of partials used in turn: one set, 115 MB, would stay in the 126 MB L2 from call to call)
    part_sets = [[(torch.randn((1, M, 12, 64), generator=g, device=dev).transpose(1, 2),
                   torch.randn((1, 12, M), generator=g, device=dev) + 20.0) for _ in range(3)] for _ in range(2)]
    merge_turn = [0]

    def merge_step():
        merge_turn[0] += 1
        return merge_attention_partials(part_sets[merge_turn[0] % 2], dt)
    steps["merge_3_partials_12500x12x64"] = (merge_step, 3 * M * 12 * 64 * 4 + 3 * M * 12 * 4 + M * 12 * 64 * 2)
    for name, (fn, nbytes) in steps.items():
        ms = _time(fn, iters)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm"], "algorithmic_bytes": nbytes}
    # a plain device copy of the RMSNorm's bytes (153.6 MB in, 153.6 MB out), timed the same way: what a launch of
    # this size reaches here (the peak in the fractions above is a copy of a much larger buffer)
    y = torch.empty_like(x)
    ms = _time(lambda: y.copy_(x), iters)
    out["rmsnorm_100000x768_bf16"]["copy_of_the_same_bytes_ms"] = ms
    out["rmsnorm_100000x768_bf16"]["frac_of_that_copy"] = ms / out["rmsnorm_100000x768_bf16"]["ms"]
    return out, steps


def side_workload(args, t5b, dev):
    """Second workloads for profiles (one GPU): see --workload."""
    peaks = measured_peaks()
    dt = torch.bfloat16
    if args.workload == "encoder":
        from turbot5_b200.t5 import T5Stack, T5StackConfig
        cfg = T5StackConfig()
        torch.manual_seed(0)
        enc = T5Stack(cfg, torch.nn.Embedding(cfg.vocab_size, cfg.d_model), is_decoder=False).to(dev).to(dt).eval()
        ids = torch.randint(0, cfg.vocab_size, (2, 8192), generator=torch.Generator().manual_seed(0)).to(dev)
        ms = _time(lambda: enc.forward_fused(ids), args.steps, warm=args.warmup)
        _emit({"metric": "t5_base_encoder_fwd_tokens_per_s", "value": 2 * 8192 / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
               "data": "synthetic", "config": {"workload": "fused T5-base encoder pass, 2 x 8192 tokens, 12 layers"}})
    else:
        res, _ = token_kernel_measurements(t5b, dev, iters=args.steps)
        _emit({"metric": "token_kernels_GBps", "value": res["add_rmsnorm_100000x768_bf16"]["GB/s"], "unit": "GB/s",
               "n_gpus": 1, "steps": args.steps, "warmup": 3, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
               "config": {"workload": "token-wise kernels at 100 000 x 768 (T5-base) bf16"},
               "roofline": {"bound": "hbm", "achieved": res["add_rmsnorm_100000x768_bf16"]["GB/s"], "peak": peaks["hbm"],
                            "unit": "GB/s", "frac": res["add_rmsnorm_100000x768_bf16"]["frac_of_hbm_peak"],
                            "kernel": "add_rmsnorm_kernel"},
               "kernels": res})


def _time(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _max_over_ranks(ms, dev, world, dist):
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _time_ranks(fn, iters, dev, world, dist, warm=1):
    """Device time of `iters` calls, barrier + synchronize on both sides, max over ranks."""
    for _ in range(warm):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    return _max_over_ranks(e0.elapsed_time(e1) / iters, dev, world, dist)


def sequence_parallel_measurement(t5b, dev, rank, world, dist):
    """One sequence of 100 000 tokens, query rows sharded over the ranks, K/V all-gathered with NCCL
    (strong scaling): one fused-bias attention layer (T5-base heads), and the whole 12-layer T5-base
    encoder with every token-wise operation on the rank's shard.  Outside the timed regions every
    rank checks rows of its own attention output against the CPU oracle on the gathered keys."""
    from oracle import t5_oracle as orc
    from turbot5_b200 import sequence_parallel as sp
    from turbot5_b200.attention import flash_attention_partial, merge_attention_partials
    from turbot5_b200.t5 import T5Stack, T5StackConfig
    L, H, D = 100000, 12, 64
    HD = H * D
    dt = torch.bfloat16
    S = sp.shard_size(L, world)
    lo, hi = sp.shard_bounds(L, world, rank)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    q = torch.randn((1, S, H, D), generator=g, device=dev, dtype=torch.float32).to(dt)
    kv = torch.randn((1, S, 2 * HD), generator=g, device=dev, dtype=torch.float32).to(dt)
    k, v = kv[..., :HD].reshape(1, S, H, D), kv[..., HD:].reshape(1, S, H, D)
    table = (torch.randn((32, H), generator=torch.Generator(device=dev).manual_seed(5), device=dev) * 0.1).to(dt)
    fl = 4.0 * H * float(L) * float(L) * D
    out = {"workload": "1 x 100000 tokens, T5-base heads (H12 D64) bf16, query rows sharded over the ranks, "
                       "K/V all-gathered per layer into local memory", "scaling": "strong",
           "all_gather_bytes_per_rank_and_layer": 0 if world == 1 else 2 * S * world * HD * 2}

    # ---- one attention layer: gather first (as before), and gather hidden behind the local keys
    ms_seq = _time_ranks(lambda: sp.sequence_parallel_attention(q, k, v, table, L, causal=False, sm_scale=1.0),
                         3, dev, world, dist)
    run_ovl = lambda: sp.sequence_parallel_attention_overlapped(q, kv, table, L, causal=False, sm_scale=1.0)
    ms_ovl = _time_ranks(run_ovl, 3, dev, world, dist)
    layer = {"ms_gather_then_attend": ms_seq, "ms_overlapped": ms_ovl, "tokens_per_s": L / (min(ms_seq, ms_ovl) * 1e-3),
             "TFLOP/s_aggregate": fl / (min(ms_seq, ms_ovl) * 1e-3) / 1e12}
    if world > 1:
        # the same kernels with no communication (keys of the other ranks already in local memory):
        # what is left of the gather outside the attention is the difference
        kv_all = torch.empty((1, world * S, 2 * HD), dtype=dt, device=dev)
        dist.all_gather_into_tensor(kv_all[0], kv[0])
        heads = lambda buf, first, a, b: buf[:, a:b, first:first + HD].unflatten(-1, (H, D)).transpose(1, 2)

        def compute_only():
            qh = q.transpose(1, 2)
            parts = [flash_attention_partial(qh, heads(kv, 0, 0, hi - lo), heads(kv, HD, 0, hi - lo), table,
                                             sm_scale=1.0, q_pos_offset=0)]
            if lo > 0:
                parts.append(flash_attention_partial(qh, heads(kv_all, 0, 0, lo), heads(kv_all, HD, 0, lo), table,
                                                     sm_scale=1.0, q_pos_offset=lo))
            if hi < L:
                parts.append(flash_attention_partial(qh, heads(kv_all, 0, hi, L), heads(kv_all, HD, hi, L), table,
                                                     sm_scale=1.0, q_pos_offset=lo - hi))
            return merge_attention_partials(parts, dt)
        ms_compute = _time_ranks(compute_only, 3, dev, world, dist)
        ms_single = _time_ranks(lambda: t5b.flash_attention_with_fusing_bias(
            q.transpose(1, 2), heads(kv_all, 0, 0, L), heads(kv_all, HD, 0, L), table, sm_scale=1.0, q_pos_offset=lo),
            3, dev, world, dist)
        layer["ms_overlapped_kernels_without_communication"] = ms_compute
        layer["ms_single_call_without_communication"] = ms_single
        layer["exposed_gather_ms_overlapped"] = ms_ovl - ms_compute
        layer["exposed_gather_ms_gather_then_attend"] = ms_seq - ms_single
    else:
        kv_all = kv
    out["one_attention_layer"] = layer

    # ---- parity of this rank's rows on the hardware path (not timed): 72 rows at the start, middle and
    # end of the shard, heads 0 and H-1, against the oracle on the gathered keys
    o_local = run_ovl()                                        # (1, S, H, D)
    torch.cuda.synchronize()
    hsel = [0, H - 1]
    k_cpu = kv_all[0, :L, :HD].view(L, H, D)[:, hsel].transpose(0, 1).unsqueeze(0).float().cpu()
    v_cpu = kv_all[0, :L, HD:].view(L, H, D)[:, hsel].transpose(0, 1).unsqueeze(0).float().cpu()
    t_cpu = table[:, hsel].float().cpu()
    n_rows, mx, mean_acc = 0, 0.0, 0.0
    real = hi - lo
    for r0 in sorted({0, max(0, real // 2 - 12), max(0, real - 24)}):
        r1 = min(r0 + 24, real)
        if r1 <= r0:
            continue
        q_cpu = q[0, r0:r1][:, hsel].transpose(0, 1).unsqueeze(0).float().cpu()
        want = orc.attention_basic(q_cpu, k_cpu, v_cpu, t_cpu, causal=False, q_pos_offset=lo + r0, slab=64)
        got = o_local[0, r0:r1][:, hsel].transpose(0, 1).unsqueeze(0).float().cpu()
        diff = (got - want).abs()
        mx = max(mx, diff.max().item())
        mean_acc += diff.mean().item() * (r1 - r0)
        n_rows += r1 - r0
    stats = torch.tensor([mx, mean_acc, float(n_rows)], dtype=torch.float64, device=dev)
    if world > 1:
        mx_t = stats[:1].clone()
        dist.all_reduce(mx_t, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        stats[0] = mx_t[0]
    out["parity"] = {"max_abs": float(stats[0]), "mean_abs": float(stats[1] / max(1.0, float(stats[2]))),
                     "rows": int(stats[2]), "heads": hsel, "tolerance": {"max_abs": 2e-2, "mean_abs": 2e-3},
                     "against": "oracle.attention_basic on the gathered keys, float32 on the CPU, every rank its own rows"}
    del kv_all, o_local

    # ---- the 12-layer T5-base encoder over the same sequence
    cfg = T5StackConfig()
    torch.manual_seed(0)
    enc = T5Stack(cfg, torch.nn.Embedding(cfg.vocab_size, cfg.d_model), is_decoder=False).to(dev).to(dt).eval()
    ids = torch.randint(0, cfg.vocab_size, (1, L), generator=torch.Generator().manual_seed(0))
    local = torch.zeros((1, S), dtype=torch.long)
    local[:, :hi - lo] = ids[:, lo:hi]
    local = local.to(dev)
    if world > 1:
        ms_enc = _time_ranks(lambda: enc.forward_fused(local, seq_len=L), 2, dev, world, dist)
        ms_enc_seq = _time_ranks(lambda: enc.forward_fused(local, seq_len=L, overlap=False), 2, dev, world, dist)
    else:
        ms_enc = ms_enc_seq = _time_ranks(lambda: enc.forward_fused(local), 2, dev, world, dist)
    gemm_fl = 2.0 * (4 * cfg.d_model * HD + 3 * cfg.d_model * cfg.d_ff) * L * cfg.num_layers
    encd = {"layers": cfg.num_layers, "ms": ms_enc, "ms_gather_then_attend": ms_enc_seq, "tokens_per_s": L / (ms_enc * 1e-3),
            "TFLOP/s_aggregate": (cfg.num_layers * fl + gemm_fl) / (ms_enc * 1e-3) / 1e12}
    if world > 1:
        # the sharded pass against the unsharded pass of the same weights on this GPU (bf16 through
        # 12 layers: compared in relative terms; the exact check of the sharding logic runs on CPU ranks)
        got = enc.forward_fused(local, seq_len=L)[0, :hi - lo].float()
        want = enc.forward_fused(ids.to(dev))[0, lo:hi].float()
        rel = ((got - want).abs().mean() / want.abs().mean()).reshape(1).double()
        dist.all_reduce(rel, op=dist.ReduceOp.MAX)
        encd["mean_rel_diff_vs_unsharded_pass"] = float(rel.item())
    out["t5_base_encoder"] = encd
    del enc
    torch.cuda.empty_cache()
    return out


def config2_measurement(t5b, dev, rank, world, dist):
    """T5-base encoder-decoder forward (12 + 12 layers, d_model 768, 12 x 64 heads, gated-GELU d_ff 2048,
    vocab 32128, random init, bf16) on 16 x 1024 encoder tokens and 16 x 128 decoder tokens; the batch is
    sharded 16 / N over the ranks with no communication.  Tokens/s = global tokens / max rank time."""
    from turbot5_b200.t5 import T5ForConditionalGeneration, T5StackConfig
    dt = torch.bfloat16
    cfg = T5StackConfig()
    torch.manual_seed(0)
    model = T5ForConditionalGeneration(cfg).to(dev).to(dt).eval()
    Bg, Le, Ld = 16, 1024, 128
    per = max(1, Bg // world)
    gcpu = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (Bg, Le), generator=gcpu)
    dec = torch.randint(0, cfg.vocab_size, (Bg, Ld), generator=gcpu)
    sl = slice((rank * per) % Bg, (rank * per) % Bg + per)
    ids_l, dec_l = ids[sl].to(dev), dec[sl].to(dev)
    with torch.no_grad():
        ms_enc = _time_ranks(lambda: model.encoder.forward_fused(ids_l), 10, dev, world, dist, warm=3)
        ms_enc_unfused = _time_ranks(lambda: model.encoder(ids_l), 10, dev, world, dist, warm=3)
        ms_full = _time_ranks(lambda: model(ids_l, dec_l), 10, dev, world, dist, warm=3)
        # the same pass as one CUDA graph (token ids copied into the graph's buffers every call)
        from turbot5_b200.t5 import GraphedForward
        graphed = GraphedForward(model, per, Le, Ld, dev)
        ms_graph = _time_ranks(lambda: graphed(ids_l, dec_l), 10, dev, world, dist, warm=3)
    n_b = per * world
    return {"workload": f"T5-base 12+12 layers bf16, {n_b} x {Le} encoder tokens + {n_b} x {Ld} decoder tokens, "
                        f"batch sharded {per} per GPU, no communication", "scaling": "strong",
            "encoder_ms": ms_enc, "encoder_tokens_per_s": n_b * Le / (ms_enc * 1e-3),
            "encoder_ms_without_fused_token_kernels": ms_enc_unfused,
            "encoder_decoder_forward_ms": ms_full,
            "encoder_decoder_tokens_per_s": n_b * (Le + Ld) / (ms_full * 1e-3),
            "encoder_decoder_forward_ms_cuda_graph": ms_graph,
            "encoder_decoder_tokens_per_s_cuda_graph": n_b * (Le + Ld) / (ms_graph * 1e-3)}


def secondary_measurements(t5b, dev):
    """Other kernels of the path at their configured sizes (inputs larger than L2 or rotated)."""
    out = {}
    dt = torch.bfloat16
    peaks = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(7)
    # token-wise kernels at 100000 x 768 bf16 (operands larger than L2)
    tk, _ = token_kernel_measurements(t5b, dev)
    out.update(tk)
    # split-KV decoding, one cross-attention layer of the T5-large decode shape: B 64, H 16, N 8192
    Bd, Hd, Nd = 64, 16, 8192
    kc = torch.randn((Bd, Hd, Nd, 64), generator=g, device=dev, dtype=torch.float32).to(dt)
    vc = torch.randn((Bd, Hd, Nd, 64), generator=g, device=dev, dtype=torch.float32).to(dt)
    qd = torch.randn((Bd, Hd, 1, 64), generator=g, device=dev, dtype=torch.float32).to(dt)
    ms = _time(lambda: t5b.flash_decoding_with_fusing_bias(qd, kc, vc, None, causal=False, sm_scale=1.0), 20)
    gbs = (2 * kc.numel() * 2) / (ms * 1e-3) / 1e9
    out["decode_cross_B64_H16_N8192"] = {"ms": ms, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm"]}
    del kc, vc
    # packed sequences: 32 sequences, lengths uniform in [128, 4096], T5-base heads
    lens = torch.randint(128, 4097, (32,), generator=torch.Generator().manual_seed(0))
    cu = torch.zeros(33, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    T = int(cu[-1])
    qkv = [torch.randn((T, 12, 64), generator=g, device=dev, dtype=torch.float32).to(dt) for _ in range(3)]
    table = (torch.randn((32, 12), generator=g, device=dev) * 0.1).to(dt)
    cu_d = cu.to(dev)
    mx = int(lens.max())
    ms = _time(lambda: t5b.flash_attention_with_fusing_bias_varlen(qkv[0], qkv[1], qkv[2], table, cu_d, cu_d, mx, mx,
                                                                   sm_scale=1.0), 20)
    fl = float((4 * 12 * 64 * lens.double() ** 2).sum())
    # host time of one call (Python wrapper + launch, no synchronisation): the reference builds its
    # work list in a Python loop with a device read per sequence on every call
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(50):
        t5b.flash_attention_with_fusing_bias_varlen(qkv[0], qkv[1], qkv[2], table, cu_d, cu_d, mx, mx, sm_scale=1.0)
    host_us = (time.perf_counter() - t0) / 50 * 1e6
    torch.cuda.synchronize()
    out["varlen_32seq_128to4096"] = {"ms": ms, "TFLOP/s": fl / (ms * 1e-3) / 1e12, "tokens": T,
                                     "frac_of_bf16_peak": fl / (ms * 1e-3) / 1e12 / peaks["tflops"],
                                     "host_us_per_call": host_us}
    del qkv
    # training step of the attention core at the headline shape: forward + backward (dQ, dK, dV and the
    # bias-table gradient).  FLOPs counted as the 5 matrix products a backward needs (2.5 x forward) plus
    # the forward; the two backward kernels recompute S and dP (7 products executed).
    qg, kg, vg = [torch.randn((2, 8192, 12, 64), generator=g, device=dev, dtype=torch.float32).to(dt)
                  .transpose(1, 2).requires_grad_(True) for _ in range(3)]
    tg = table.detach().clone().requires_grad_(True)
    dout = torch.randn((2, 12, 8192, 64), generator=g, device=dev, dtype=torch.float32).to(dt)

    def train_step():
        o_ = t5b.flash_attention_with_fusing_bias(qg, kg, vg, tg, sm_scale=1.0)
        o_.backward(dout)
    ms = _time(train_step, 10)
    with torch.no_grad():
        ms_f = _time(lambda: t5b.flash_attention_with_fusing_bias(qg, kg, vg, tg, sm_scale=1.0), 10)
    fl = 4.0 * 2 * 12 * 8192 * 8192 * 64
    out["attention_fwd_bwd_B2_H12_L8192"] = {"ms_fwd_bwd": ms, "ms_fwd": ms_f, "ms_bwd": ms - ms_f,
                                             "TFLOP/s_fwd_bwd": 3.5 * fl / (ms * 1e-3) / 1e12,
                                             "TFLOP/s_bwd": 2.5 * fl / ((ms - ms_f) * 1e-3) / 1e12,
                                             "frac_of_bf16_peak_bwd": 2.5 * fl / ((ms - ms_f) * 1e-3) / 1e12 / peaks["tflops"]}
    del qg, kg, vg, tg, dout
    # RMSNorm backward, 100000 x 768 bf16: reads x and dy, writes dx (3 x 154 MB) + the weight gradient;
    # timed at the C ABI (the autograd wrapper adds a zero-fill and a cast of the 768 weight gradients)
    from turbot5_b200 import _native as nat
    xg = torch.randn((100000, 768), generator=g, device=dev).to(dt)
    wg = torch.rand((768,), generator=g, device=dev).to(dt)
    dyg = torch.randn((100000, 768), generator=g, device=dev).to(dt)
    dxg, dwg = torch.empty_like(xg), torch.zeros((768,), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    ms = _time(lambda: nat.check(nat.lib().t5b_rmsnorm_bwd(xg.data_ptr(), wg.data_ptr(), dyg.data_ptr(), dxg.data_ptr(),
                                                           dwg.data_ptr(), 100000, 768, 768, 768, 768, nat.BF16, nat.BF16,
                                                           1e-6, stream), "rmsnorm bwd"), 30)
    gbs = 3 * xg.numel() * 2 / (ms * 1e-3) / 1e9
    out["rmsnorm_bwd_100000x768_bf16"] = {"ms": ms, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm"]}
    del xg, wg, dyg, dxg
    # block-local attention (T5LocalAttention): 1 x 12 heads x 65536 tokens, blocks of 512 rows, each seeing
    # 3 x 512 keys: FLOPs counted over the visible window only
    ql, kl, vl_ = [torch.randn((1, 65536, 12, 64), generator=g, device=dev, dtype=torch.float32).to(dt).transpose(1, 2)
                   for _ in range(3)]
    ms = _time(lambda: t5b.flash_attention_with_fusing_bias(ql, kl, vl_, table, sm_scale=1.0, local_block=512), 20)
    fl = 4.0 * 12 * 65536 * (3 * 512) * 64
    out["local_attention_H12_L65536_block512"] = {"ms": ms, "TFLOP/s": fl / (ms * 1e-3) / 1e12,
                                                  "tokens_per_s": 65536 / (ms * 1e-3),
                                                  "frac_of_bf16_peak": fl / (ms * 1e-3) / 1e12 / peaks["tflops"]}
    del ql, kl, vl_
    # head dim 128 (the T5-3B / 11B head size): same sequence length, 3 rotating input sets
    # (3 x 151 MB > L2), T5 bias, bf16
    sets = [[(torch.randn((2, 8192, 12, 128), generator=g, device=dev, dtype=torch.float32) * 0.5).to(dt).transpose(1, 2)
             for _ in range(3)] for _ in range(3)]
    turn = [0]

    def d128_step():
        q_, k_, v_ = sets[turn[0] % 3]
        turn[0] += 1
        return t5b.flash_attention_with_fusing_bias(q_, k_, v_, table, sm_scale=1.0)
    ms = _time(d128_step, 15)
    fl = 4.0 * 2 * 12 * 8192 * 8192 * 128
    out["attention_d128_B2_H12_L8192"] = {"ms": ms, "TFLOP/s": fl / (ms * 1e-3) / 1e12,
                                          "frac_of_bf16_peak": fl / (ms * 1e-3) / 1e12 / peaks["tflops"]}
    del sets
    # T5-base encoder (12 layers, d_model 768, 12 x 64 heads, gated-GELU d_ff 2048, random init, bf16):
    # tokens/s of a forward pass at 2 x 8192 tokens and at 16 x 1024 tokens
    from turbot5_b200.t5 import T5Stack, T5StackConfig
    cfg = T5StackConfig()
    torch.manual_seed(0)
    enc = T5Stack(cfg, torch.nn.Embedding(cfg.vocab_size, cfg.d_model), is_decoder=False).to(dev).to(dt).eval()
    for Bt, Lt in ((2, 8192), (16, 1024)):
        ids = torch.randint(0, cfg.vocab_size, (Bt, Lt), generator=g, device=dev)
        with torch.no_grad():
            ms = _time(lambda: enc.forward_fused(ids), 5, warm=2)
            ms_mod = _time(lambda: enc(ids), 5, warm=2)
        out[f"t5_base_encoder_fwd_{Bt}x{Lt}"] = {"ms": ms, "tokens_per_s": Bt * Lt / (ms * 1e-3),
                                                 "ms_without_fused_token_kernels": ms_mod}
    # a padded batch: 16 x 1024 with lengths uniform in [128, 1024].  The module path unpads and pads around every
    # attention call and runs everything else on the padded batch; the fused pass packs the valid tokens once.
    lens = torch.randint(128, 1025, (16,), generator=torch.Generator().manual_seed(1))
    mask = (torch.arange(1024)[None, :] < lens[:, None]).to(torch.int64).to(dev)
    n_tok = int(lens.sum())
    with torch.no_grad():
        ms_mod = _time(lambda: enc(ids, attention_mask=mask), 5, warm=2)
        ms_packed = _time(lambda: enc.forward_fused(ids, attention_mask=mask), 5, warm=2)
        ms_packed_known = _time(lambda: enc.forward_fused(ids, attention_mask=mask, packed_rows=n_tok), 5, warm=2)
    out["t5_base_encoder_fwd_16x1024_padded"] = {
        "valid_tokens": n_tok, "ms_module_path": ms_mod, "ms_packed_once": ms_packed,
        "ms_packed_once_token_count_known": ms_packed_known, "valid_tokens_per_s": n_tok / (ms_packed * 1e-3)}
    del enc
    # the same encoder with block-local self-attention (blocks of 512) over one 65 536-token sequence
    cfg_l = T5StackConfig(attention_type="local", sliding_window=512)
    enc = T5Stack(cfg_l, torch.nn.Embedding(cfg_l.vocab_size, cfg_l.d_model), is_decoder=False).to(dev).to(dt).eval()
    ids = torch.randint(0, cfg_l.vocab_size, (1, 65536), generator=g, device=dev)
    with torch.no_grad():
        ms = _time(lambda: enc(ids), 5, warm=2)
    out["t5_base_local_encoder_fwd_1x65536"] = {"ms": ms, "tokens_per_s": 65536 / (ms * 1e-3)}
    del enc
    # T5-large-shaped greedy decoding (24 decoder layers, d_model 1024, 16 x 64 heads, d_ff 4096 ReLU as in
    # the original T5-large; random init, bf16): batch 64 against an encoder memory of 8192 states.  Every
    # step streams the cross-attention K/V of all layers (51.5 GB) through the split-KV kernel.
    try:
        from turbot5_b200.t5 import T5ForConditionalGeneration
        free, _ = torch.cuda.mem_get_info(dev)
        if free > 90e9:
            cfg5 = T5StackConfig(d_model=1024, d_kv=64, d_ff=4096, num_layers=0, num_decoder_layers=24, num_heads=16,
                                 feed_forward_proj="relu")
            model = T5ForConditionalGeneration(cfg5).to(dev).to(dt).eval()
            enc_states = torch.randn((64, 8192, 1024), generator=g, device=dev, dtype=torch.float32).to(dt)
            with torch.no_grad():
                cache = model.decoder.new_cache(enc_states, 40)
                cur = torch.zeros((64, 1), dtype=torch.long, device=dev)
                for _ in range(4):                      # warm-up steps
                    cur = model.logits(model.decoder.decode_step(cur, cache))[:, -1:].argmax(-1)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                steps = 32
                e0.record()
                for _ in range(steps):
                    cur = model.logits(model.decoder.decode_step(cur, cache))[:, -1:].argmax(-1)
                e1.record()
                torch.cuda.synchronize()
            ms_eager = e0.elapsed_time(e1) / steps
            del cache
            # the same step as one CUDA graph per token
            from turbot5_b200.t5 import GraphedDecoding
            session = GraphedDecoding(model, enc_states, 40)
            for _ in range(4):
                session.step()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                session.step()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            cache = session
            kv_bytes = 24 * 2 * 64 * 16 * 8192 * 64 * 2
            out["t5_large_decode_B64_enc8192"] = {"ms_per_step": ms, "ms_per_step_without_cuda_graph": ms_eager,
                                                  "tokens_per_s": 64 / (ms * 1e-3),
                                                  "cross_kv_GB_per_step": kv_bytes / 1e9,
                                                  "GB/s_cross_kv_only": kv_bytes / (ms * 1e-3) / 1e9,
                                                  "frac_of_hbm_peak": kv_bytes / (ms * 1e-3) / 1e9 / peaks["hbm"]}
            del model, cache, enc_states
    except torch.cuda.OutOfMemoryError:
        out["t5_large_decode_B64_enc8192"] = {"skipped": "not enough free device memory"}
    return out


if __name__ == "__main__":
    main()
