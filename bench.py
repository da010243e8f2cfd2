"""Benchmark of the Clef-Omni MoE block on B200: MoE-layer prefill tokens/s at T=4096.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the block (router -> top-8 -> permutation -> gate/up+SwiGLU -> down ->
combine) over one packed batch.  Workload at N=1: BASELINE configuration 2 -- T=4096 as eight
packed sequences (lengths uniform in [64,1024] rescaled to 4096), hidden 2048, 128 experts
top-8, intermediate 768, BF16 weights N(0,0.02), BF16 activations N(0,1), seed 1.

Prints ONE JSON line.  `value` is tokens/s with inputs resident in HBM; `e2e` is the same
metric through the host-buffer C-ABI call with the copies inside the timed region; `roofline`
is the gate/up expert product (the dominant kernel) against the measured BF16 peak;
`cpu_baseline` is the PyTorch CPU block the reference's Python oracle runs, timed on a bounded
sample of the same workload on this host.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

T_TOKENS = 4096          # overridden by --tokens for small profiling captures
SEED = 1
H, F, E, TOP = 2048, 768, 128, 8
GATEUP_FLOP_PER_TOKEN = 2 * H * (2 * F) * TOP          # 50,331,648
EXPERT_FLOP_PER_TOKEN = GATEUP_FLOP_PER_TOKEN + 2 * F * H * TOP   # 75,497,472
WEIGHT_BYTES = (E * H + E * 2 * F * H + E * H * F) * 2
KERNELS_PER_PASS = 7     # router (counts the sort segments), exact pass, scan, scatter, gate/up (gathers its rows), down, combine
KERNELS_PER_PASS_EP = 12 # ... plus plan, dispatch, return and two barriers
METRIC = "MoE-layer prefill tokens/sec at T=4096"
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch at T=4096, from the ncu
# capture summarised in profiles/ncu_full_router_experts_combine_T4096.md
GATEUP_DRAM_TRAFFIC_T4096 = 964_327_424 + 43_772_928


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(bf16_tflops=float(d["bf16_tflops"]), bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=reasons,
                    samples=len(sm))


def cpu_block(router, gate_up, down):
    """The CPU block the reference's Python oracle executes per layer (ref/omni.py:125-128):
    Hugging Face Qwen3OmniMoeThinkerTextSparseMoeBlock, eager experts, FP32 math on the
    BF16-rounded weights.  Falls back to the FP32 port in oracle/ when transformers lacks it."""
    import torch
    try:
        from transformers.models.qwen3_omni_moe import modeling_qwen3_omni_moe as m
        from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeTextConfig
        cfg = Qwen3OmniMoeTextConfig(hidden_size=H, moe_intermediate_size=F, num_experts=E, num_experts_per_tok=TOP,
                                     norm_topk_prob=True)
        cfg._experts_implementation = "eager"
        blk = m.Qwen3OmniMoeThinkerTextSparseMoeBlock(cfg).eval()
        with torch.no_grad():
            blk.gate.weight.copy_(router.float())
            blk.experts.gate_up_proj.copy_(gate_up.float())
            blk.experts.down_proj.copy_(down.float())

        def run(x):
            with torch.inference_mode():
                y = blk(x[None])
                return y[0] if isinstance(y, tuple) else y
        return run, "reference", "Hugging Face Qwen3OmniMoeThinkerTextSparseMoeBlock (the block ref/omni.py runs), FP32 on BF16-rounded weights"
    except Exception:   # pragma: no cover - depends on the installed transformers
        from oracle import omni_oracle as orc

        def run(x):
            with torch.inference_mode():
                return orc.moe_block_f32(x, router, gate_up, down)[0]
        return run, "port", "FP32 restatement of the block (oracle/omni_oracle.py: moe_block_f32)"


def time_cpu(run, x, steps, warmup):
    for _ in range(warmup):
        run(x)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        run(x)
        times.append(time.perf_counter() - t0)
    return times


def reference_arm(args):
    """The reference's own CPU implementation of the path on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from cleffa_b200 import workloads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    router, gate_up, down = workloads.make_weights(SEED)
    x = workloads.make_activations(SEED, T_TOKENS).float()
    run, kind, what = cpu_block(router, gate_up, down)
    probe = time_cpu(run, x[:512].contiguous(), 1, 1)[0]
    budget = 150.0 / max(1, args.steps + args.warmup)
    sample_t = T_TOKENS if probe * (T_TOKENS / 512) <= budget else 512
    xs = x[:sample_t].contiguous()
    times = time_cpu(run, xs, args.steps, max(1, args.warmup))
    total = sum(times)
    value = sample_t * args.steps / total
    sample = f"{what}; first {sample_t} of {T_TOKENS} tokens per step, {torch.get_num_threads()} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(1), "tokens": sample_t},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_name(n_gpus):
    return (f"Clef-Omni MoE layer, T={T_TOKENS} packed varlen prefill (8 sequences), hidden 2048, 128 experts top-8, "
            f"intermediate 768, bf16 weights N(0,0.02), bf16 activations N(0,1), seed {SEED}"
            + ("" if n_gpus == 1 else f", per GPU (experts sharded {E // n_gpus} per GPU)"))


def ours(args):
    import torch
    import torch.distributed as dist
    from cleffa_b200 import OmniBackend, workloads

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    router, gate_up, down = workloads.make_weights(SEED)
    x_host = workloads.make_activations(SEED + 1000 * rank, T_TOKENS).pin_memory()
    bounds = workloads.varlen_bounds(SEED, T_TOKENS)
    res_host = torch.zeros(T_TOKENS, H).pin_memory()

    # Dedicated streams: the library launches on them and the timing events are recorded on the
    # main one (the legacy default stream has handle 0, which the C-ABI reads as "create your own").
    # With expert parallelism the tokens of a rank are split into `micro` independent
    # micro-batches, each driven through its own library context and stream, so that one
    # micro-batch's peer transfers overlap the other's expert products.
    micro = max(1, args.micro if args.micro else 1)
    main_stream = torch.cuda.Stream()
    torch.cuda.set_stream(main_stream)
    streams = [main_stream] + [torch.cuda.Stream() for _ in range(micro - 1)]
    bs = [OmniBackend(local, stream=st.cuda_stream) for st in streams]
    for b in bs:
        b.reserve(T_TOKENS)
        for kv in args.option:                           # library options, name=value (for A/B runs)
            name, _, val = kv.partition("=")
            b.set_option(name, int(val))
    if world > 1:
        # expert parallel: 128/world experts per GPU; every rank maps every rank's exchange buffers
        el = E // world
        dev_w = (router.cuda(), gate_up[rank * el:(rank + 1) * el].cuda(), down[rank * el:(rank + 1) * el].cuda())
        for b in bs:
            handles = [None] * world
            dist.all_gather_object(handles, b.ep_export())
            b.ep_connect(rank, world, b"".join(handles))
            b.bind_layer(0, *dev_w)                      # one device copy of the rank's expert slice, shared
        dist.barrier()                                   # every rank has mapped every rank
        for b in bs:
            b.ep_sync(30000)                             # first touch of the peers' memory happens here
        for bi in bs:
            if args.reserve:
                bi.set_option("reserve_sms", args.reserve)
            if args.overlap:
                bi.set_option("ep_overlap", 1)   # room for the other micro-batch's small kernels
        if micro > 1 and not args.no_gate:
            # stagger the micro-batches: context i starts its dispatch when context i-1 finished its own,
            # so one micro-batch's transfers run under the other's expert products instead of in lock-step
            gates = [torch.cuda.Event() for _ in range(micro)]
            for i, (ev, st) in enumerate(zip(gates, streams)):
                ev.record(st)                            # gives every event a handle; the first waits pass
            torch.cuda.synchronize()
            for i, bi in enumerate(bs):
                bi.ep_gate(gates[(i - 1) % micro].cuda_event, gates[i].cuda_event)
    else:
        bs[0].bind_layer(0, router, gate_up, down)
    b = bs[0]
    n_layers = max(1, args.layers)
    if n_layers > 1:
        # BASELINE configuration 3 on one GPU: a stack of MoE sublayers, each followed by the
        # residual add, independent random-init weights per layer generated on the device
        if world != 1:
            raise SystemExit("--layers needs --gpus 1")
        b.reserve(T_TOKENS, n_layer=n_layers)
        g = torch.Generator(device="cuda").manual_seed(SEED)
        stack = []
        for l in range(1, n_layers):
            wl = tuple((torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                       for shape in ((E, H), (E, 2 * F, H), (E, H, F)))
            b.bind_layer(l, *wl)
            stack.append(wl)
        if args.norm:
            for l in range(n_layers):
                b.bind_norm(l, torch.ones(H), 1e-6)
    xn = x_host.cuda()
    x = torch.zeros(T_TOKENS, H, device="cuda")
    x0 = xn.float() if n_layers > 1 else None
    cuts = [T_TOKENS * i // micro for i in range(micro + 1)]
    torch.cuda.synchronize()

    def step():
        if n_layers > 1:
            b.begin()
            x.copy_(x0)                         # every step starts from the same N(0,1) residual stream
            for l in range(n_layers):
                if args.norm:
                    b.encode_norm_moe(l, x, bounds)     # RMSNorm of the residual stream inside the library
                else:
                    xn.copy_(x)                 # FP32 residual -> BF16 layer input (the norm's place)
                    b.encode_moe(l, xn, x, bounds)
            return
        if micro == 1:
            b.begin()
            b.encode_moe(0, xn, x, bounds)
            return
        for i, bi in enumerate(bs):
            bi.begin()
            bi.encode_moe(0, xn[cuts[i]:cuts[i + 1]], x[cuts[i]:cuts[i + 1]])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    for _ in range(max(3, args.warmup)):
        step()
    for bi in bs:
        bi.complete()

    # ---- device-resident timing.  Two timed regions of the same K steps: the first gives
    # `value`; the second repeats it with a CUDA event recorded between the stages of every pass
    # and gives the per-kernel durations for the roofline.  The marks are kept out of the first
    # region because they cost about 20 us per pass and stop a kernel's prologue from
    # overlapping the previous kernel's tail.
    def timed_region():
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as sampler:
            start.record(main_stream)
            for st in streams[1:]:
                st.wait_event(start)
            for _ in range(args.steps):
                step()
            for st in streams[1:]:
                done = torch.cuda.Event()
                done.record(st)
                main_stream.wait_event(done)
            stop.record(main_stream)
            barrier()
        for bi in bs:
            bi.complete()
        return start.elapsed_time(stop), sampler

    elapsed_ms, clocks = timed_region()
    if args.kernels_only and world == 1:
        # for captures under a profiler: the warm-up and the K timed steps, nothing else
        if rank == 0:
            print(json.dumps({"kernels_only": True, "ms_per_step": elapsed_ms / args.steps, "tokens": T_TOKENS, "n_gpus": world}))
        for bi in bs:
            bi.close()
        return
    b.set_option("profile", 1)
    marked_ms, _ = timed_region()
    stages = b.profile()
    b.set_option("profile", 0)
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t[0])
    clock_summary = clocks.summary()
    if clock_summary["samples"] < 5:
        # K steps last a few milliseconds, less than one nvidia-smi sample: keep the same loop
        # running for about a second (untimed) so that the clocks under this load are seen.
        # The number of passes is derived from the agreed step time: every rank runs the same count.
        probe_passes = int(min(5000, max(20, 1000.0 / max(elapsed_ms / args.steps, 1e-3))))
        with ClockSampler(local) as probe:
            for i in range(probe_passes):
                step()
                if i % 20 == 19:
                    for bi in bs:
                        bi.complete()
            for bi in bs:
                bi.complete()
        clock_summary = dict(probe.summary(), note="sampled over an untimed continuation of the timed loop (about 1 s)")

    # ---- end to end through the host-buffer call (copies inside the timed region)
    for _ in range(2):
        b.forward_host(0, x_host, res_host, bounds)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        b.forward_host(0, x_host, res_host, bounds)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t[0])

    if rank == 0:
        peaks = measured_peaks()
        tokens = T_TOKENS * world
        value = tokens * args.steps / (elapsed_ms * 1e-3)
        gateup_ms = stages["gate_up"]
        achieved = GATEUP_FLOP_PER_TOKEN * T_TOKENS / (gateup_ms * 1e-3) / 1e12 if gateup_ms > 0 else 0.0
        both_ms = stages["gate_up"] + stages["down"]
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(world) + (f", {n_layers} stacked layers with residual adds, weights generated on the device" if n_layers > 1 else ""), "parallelism": "single GPU" if world == 1 else f"expert parallel ep{world}, tokens data-parallel, peer-store dispatch/return over NVLink, {micro} micro-batches per rank on separate streams", "l2": "each step streams 1.21 GB of expert weights (> 126 MB L2); no explicit flush",
                       "timing": "CUDA events on the launching stream, max over ranks"},
            "e2e": {"value": tokens * args.steps / e2e_s, "unit": "tokens/s",
                    "h2d_bytes_per_step": T_TOKENS * H * 2 + T_TOKENS * H * 4, "d2h_bytes_per_step": T_TOKENS * H * 4},
            "gpu_launches": ((KERNELS_PER_PASS + (1 if args.norm else 0)) * n_layers if world == 1 else KERNELS_PER_PASS_EP * micro) * args.steps,
            "clocks": clock_summary,
            "roofline": {"bound": "tensor", "kernel": "expert_gemm_kernel<gate_up+SwiGLU>", "achieved": achieved,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                         "peak_source": peaks["source"] + " (burst cuBLAS bf16 figure; the kernel runs under sw_power_cap, for which the sustained figure is the like-for-like one)",
                         "peak_sustained": peaks["bf16_tflops_sustained"], "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                         "traffic": GATEUP_DRAM_TRAFFIC_T4096 if (T_TOKENS == 4096 and world == 1) else None,
                         # gate/up weights once, every token row once (the kernel gathers them), h written once
                         "algorithmic_bytes": E * 2 * F * H * 2 + T_TOKENS * H * 2 + T_TOKENS * TOP * F * 2},
            "stages_ms": stages,
            "stages_note": f"from a second timed region of the same {args.steps} steps with an event recorded between stages ({marked_ms / args.steps:.4f} ms per step)",
            "expert_gemms": {"tflops": EXPERT_FLOP_PER_TOKEN * T_TOKENS / (both_ms * 1e-3) / 1e12 if both_ms > 0 else 0.0,
                             "frac_of_bf16_peak": (EXPERT_FLOP_PER_TOKEN * T_TOKENS / (both_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]) if both_ms > 0 else 0.0,
                             "frac_of_sustained_bf16_peak": (EXPERT_FLOP_PER_TOKEN * T_TOKENS / (both_ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"]) if both_ms > 0 else 0.0},
            "hbm": {"weights_gbs_over_layer": WEIGHT_BYTES / (elapsed_ms / args.steps * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"]},
        }
        if world == 1 and not args.no_cpu:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            run, kind, what = cpu_block(router, gate_up, down)
            xs = x_host[:512].float().contiguous()
            times = time_cpu(run, xs, 3, 1)
            line["cpu_baseline"] = {"value": 512 / min(times), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                                    "sample": f"{what}; first 512 of {T_TOKENS} tokens, best of 3 after one warm-up"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        for bi in bs:
            bi.ep_disconnect()
        dist.barrier()
    for bi in bs:
        bi.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    global T_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU (default: the headline 4096)")
    ap.add_argument("--no-gate", action="store_true", help="do not stagger the micro-batches")
    ap.add_argument("--reserve", type=int, default=0, help="SMs the expert kernels leave to the copy kernels with expert parallelism (0: the library default, 32)")
    ap.add_argument("--norm", action="store_true", help="with --layers: each layer normalises the residual stream itself (RMSNorm, unit weights) instead of taking a BF16 copy")
    ap.add_argument("--kernels-only", action="store_true", help="run the warm-up and the timed steps and stop (for profiler captures; one GPU)")
    ap.add_argument("--option", action="append", default=[], help="library option name=value (clef_omni_set_option), repeatable")
    ap.add_argument("--overlap", action="store_true", help="expert parallelism: run the transfers under the expert kernels")
    ap.add_argument("--layers", type=int, default=1, help="stack of MoE sublayers with residual adds (one GPU; BASELINE configuration 3 uses 48 at --tokens 16384)")
    ap.add_argument("--micro", type=int, default=0, help="micro-batches per rank, each on its own context and stream (default 1)")
    args = ap.parse_args()
    T_TOKENS = args.tokens
    if args.impl == "reference":
        reference_arm(args)
    else:
        ours(args)


if __name__ == "__main__":
    main()
