"""Benchmark of the Clef-Omni MoE block on B200: MoE-layer prefill tokens/s at T=4096.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the block (router -> top-8 -> permutation -> gate/up+SwiGLU -> down ->
combine) over one packed batch.  Workload at N=1: BASELINE configuration 2 -- T=4096 as eight
packed sequences (lengths uniform in [64,1024] rescaled to 4096), hidden 2048, 128 experts
top-8, intermediate 768, BF16 weights N(0,0.02), BF16 activations N(0,1), seed 1.

Prints ONE JSON line.  `value` is tokens/s with inputs resident in HBM; `e2e` is the same
metric through the host-buffer C-ABI call with the copies inside the timed region; `roofline`
is the gate/up expert product (the dominant kernel) against the measured BF16 peak;
`cpu_baseline` is the PyTorch CPU block the reference's Python oracle runs, timed on this host.

The K-step timed region is repeated until at least one second of device time has been timed;
`ms_per_step` is the median region (min and max beside it) and `clocks` are the nvidia-smi
samples taken while those regions ran.

Other workloads of BASELINE.json (each prints one JSON line of the same shape):
    --layers 48 --tokens 16384 [--strong --gpus N]   configuration 3, the 48-layer stack
    --bias zipf --tokens 8192 [--strong --gpus N]    configuration 4, Zipf-skewed routing
    --sweep                                          configuration 5, T = 1 .. 256 latency table
With --strong the token count is the whole job's and every rank takes 1/N of it (strong
scaling); without it, it is per GPU (weak scaling, the default the headline uses).
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
KERNELS_PER_PASS_EP = 10  # ... plus owner buckets, plan and one barrier; the expert kernels dispatch and return the rows themselves
METRIC = "MoE-layer prefill tokens/sec at T=4096"
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch at T=4096, from the ncu
# capture summarised in profiles/ncu_full_moe_layer_T4096.md
GATEUP_DRAM_TRAFFIC_T4096 = 864_723_456 + 46_342_144


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


def cpu_reference(T, steps, warmup):
    """Times the reference's CPU block on this host: all T tokens per step when a probe says the
    run fits the budget (else the first 512), every host core, mean over the steps.  The GPU
    arm's `cpu_baseline` and the reference arm both come from here, so they agree."""
    import torch
    from cleffa_b200 import workloads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    router, gate_up, down = workloads.make_weights(SEED)
    x = workloads.make_activations(SEED, T).float()
    run, kind, what = cpu_block(router, gate_up, down)
    probe_t = min(512, T)
    probe = time_cpu(run, x[:probe_t].contiguous(), 1, 1)[0]
    budget = 150.0 / max(1, steps + warmup)
    sample_t = T if probe * (T / probe_t) <= budget else probe_t
    xs = x[:sample_t].contiguous()
    times = time_cpu(run, xs, steps, max(1, warmup))
    total = sum(times)
    return dict(value=sample_t * steps / total, ms_per_step=1e3 * total / steps, tokens=sample_t, kind=kind, cores=torch.get_num_threads(),
                sample=f"{what}; first {sample_t} of {T} tokens per step, mean of {steps} steps after {max(1, warmup)} warm-up, "
                       f"{torch.get_num_threads()} threads")


def reference_arm(args):
    """The reference's own CPU implementation of the path on this host's cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    r = cpu_reference(T_TOKENS, args.steps, args.warmup)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(1), "tokens": r["tokens"]},
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_name(n_gpus, args=None):
    strong = bool(args and args.strong)
    layers = max(1, args.layers) if args else 1
    zipf = bool(args and args.bias == "zipf")
    shape = "packed varlen prefill (8 sequences)" if not (zipf or layers > 1) else "one sequence"
    name = (f"Clef-Omni MoE layer, T={T_TOKENS} {shape}, hidden 2048, 128 experts top-8, "
            f"intermediate 768, bf16 weights N(0,0.02), bf16 activations N(0,1), seed {SEED}")
    if zipf:
        name += ", router logits + 2 ln(Zipf(1.2)) bias over a random expert permutation"
    if layers > 1:
        name += f", {layers} stacked layers with residual adds, independent weights generated on the device"
    if n_gpus > 1:
        name += (f", {T_TOKENS} tokens over {n_gpus} GPUs" if strong else ", per GPU") + f" (experts sharded {E // n_gpus} per GPU)"
    return name


def regime(clock_summary):
    """Which measured BF16 peak is the like-for-like one for the clocks seen while timing."""
    if "sw_power_cap" in (clock_summary.get("reasons") or []):
        return "sustained (sw_power_cap active while the timed regions ran, as in the seconds-long cuBLAS loop)"
    return "burst (no power cap seen while the timed regions ran)"


def ours(args):
    import numpy as np
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

    # tokens of this rank: the whole job's T split evenly (strong scaling) or T per GPU (weak)
    if args.strong and T_TOKENS % world:
        raise SystemExit("--strong needs a token count divisible by the number of GPUs")
    T = T_TOKENS // world if args.strong else T_TOKENS
    n_layers = max(1, args.layers)
    zipf = args.bias == "zipf"
    single_seq = zipf or n_layers > 1
    el = E // world
    router, gate_up, down = workloads.make_weights(SEED)
    bias = torch.from_numpy(workloads.zipf_bias(SEED)) if zipf else None
    if args.strong:
        x_host = workloads.make_activations(SEED, T_TOKENS)[rank * T:(rank + 1) * T].contiguous().pin_memory()
    else:
        x_host = workloads.make_activations(SEED + 1000 * rank, T).pin_memory()
    bounds = np.array([0, T], np.int32) if (single_seq or args.strong) else workloads.varlen_bounds(SEED, T)
    res_host = torch.zeros(T, H).pin_memory()

    # A dedicated stream: the library launches on it and the timing events are recorded on it
    # (the legacy default stream has handle 0, which the C-ABI reads as "create your own").
    main_stream = torch.cuda.Stream()
    torch.cuda.set_stream(main_stream)
    b = OmniBackend(local, stream=main_stream.cuda_stream)
    b.reserve(T, n_layer=n_layers)
    for kv in args.option:                               # library options, name=value (for A/B runs)
        name, _, val = kv.partition("=")
        b.set_option(name, int(val))

    def layer_weights(l):
        """Layer 0: the seeded host weights.  Further layers: generated on the device from a seed
        every rank shares, so that each rank can keep just its expert slice."""
        if l == 0:
            return router, gate_up, down
        g = torch.Generator(device="cuda").manual_seed(1000 * SEED + l)
        return tuple((torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                     for shape in ((E, H), (E, 2 * F, H), (E, H, F)))

    if world > 1:
        # expert parallel: 128/world experts per GPU; every rank maps every rank's exchange buffers
        handles = [None] * world
        dist.all_gather_object(handles, b.ep_export())
        b.ep_connect(rank, world, b"".join(handles))
        for l in range(n_layers):
            r_, gu_, dn_ = layer_weights(l)
            b.bind_layer(l, r_.cuda(), gu_[rank * el:(rank + 1) * el].cuda().contiguous(), dn_[rank * el:(rank + 1) * el].cuda().contiguous(),
                         bias=bias.cuda() if bias is not None else None)
            del r_, gu_, dn_
        dist.barrier()                                   # every rank has mapped every rank
        b.ep_sync(30000)                                 # first touch of the peers' memory happens here
    else:
        b.bind_layer(0, router, gate_up, down, bias=bias)
        for l in range(1, n_layers):
            b.bind_layer(l, *layer_weights(l))
    if args.norm:
        for l in range(n_layers):
            b.bind_norm(l, torch.ones(H), 1e-6)
    xn = x_host.cuda()
    x = torch.zeros(T, H, device="cuda")
    x0 = xn.float() if n_layers > 1 else None
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
        b.begin()
        b.encode_moe(0, xn, x, bounds)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(v, op):
        """max or min of a host number over the ranks"""
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t[0])

    barrier()
    for _ in range(max(3, args.warmup)):
        step()
    b.complete()

    def timed_region():
        """EXACTLY `steps` steps between two events on the launching stream, bracketed by a
        barrier and a device synchronize on both sides.  Returns the max over ranks (ms)."""
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(main_stream)
        for _ in range(args.steps):
            step()
        stop.record(main_stream)
        barrier()
        b.complete()
        ms = start.elapsed_time(stop)
        return agree(ms, dist.ReduceOp.MAX) if world > 1 else ms

    # ---- device-resident timing: the K-step region is repeated until >= 1 s of device time has
    # been timed (every rank runs the same number of regions: the count is agreed after each).
    regions = []
    with ClockSampler(local) as sampler:
        while True:
            regions.append(timed_region())
            enough = sum(regions) >= args.min_time_ms or len(regions) >= args.max_regions
            if agree(1.0 if enough else 0.0, dist.ReduceOp.MAX if world > 1 else None) > 0:
                break
    elapsed_ms = statistics.median(regions)
    clock_summary = dict(sampler.summary(), note=f"sampled every 100 ms while the {len(regions)} timed regions ran "
                                                f"({sum(regions) / 1e3:.2f} s of device time)")
    if args.kernels_only and world == 1:
        # for captures under a profiler: the warm-up and the timed steps, nothing else
        print(json.dumps({"kernels_only": True, "ms_per_step": elapsed_ms / args.steps, "tokens": T, "n_gpus": world}))
        b.close()
        return

    # ---- a further region of the same K steps with an event recorded between the stages of every
    # pass: per-kernel durations for the roofline.  Kept out of the regions above because the
    # marks cost about 20 us per pass and stop a kernel's prologue from overlapping the previous
    # kernel's tail -- the marked stages therefore sum to MORE than ms_per_step.
    b.set_option("profile", 1)
    marked_ms = timed_region()
    stages = b.profile()
    b.set_option("profile", 0)

    # ---- expert parallelism: one untimed, checked pass.  Every rank runs its own tokens through a
    # second, single-GPU context holding all 128 experts of layer 0 and compares the bytes.
    ep_equal = None
    if world > 1:
        out_ep = torch.zeros(T, H, device="cuda")
        b.begin(); b.encode_moe(0, xn, out_ep, bounds); b.complete()
        solo_stream = torch.cuda.Stream()
        with OmniBackend(local, stream=solo_stream.cuda_stream) as solo:
            solo.reserve(T)
            solo.bind_layer(0, router, gate_up, down, bias=bias)
            out_1 = torch.zeros(T, H, device="cuda")
            torch.cuda.synchronize()
            solo.begin(); solo.encode_moe(0, xn, out_1, bounds); solo.complete()
        ep_equal = agree(1.0 if torch.equal(out_ep, out_1) else 0.0, dist.ReduceOp.MIN) > 0

    # ---- end to end through the host-buffer call (copies inside the timed region), layer 0
    for _ in range(2):
        b.forward_host(0, x_host, res_host, bounds)
    e2e_regions = []
    while True:
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            b.forward_host(0, x_host, res_host, bounds)
        torch.cuda.synchronize()
        e2e_regions.append(agree(time.perf_counter() - t0, dist.ReduceOp.MAX if world > 1 else None))
        enough = sum(e2e_regions) >= args.min_time_ms / 2e3 or len(e2e_regions) >= args.max_regions
        if agree(1.0 if enough else 0.0, dist.ReduceOp.MAX if world > 1 else None) > 0:
            break
    e2e_s = statistics.median(e2e_regions)

    if rank == 0:
        peaks = measured_peaks()
        tokens = T * world
        value = tokens * args.steps / (elapsed_ms * 1e-3)
        per_layer = 1.0 / n_layers                      # stage marks are means over all passes (= layers)
        gateup_ms = stages["gate_up"]
        achieved = GATEUP_FLOP_PER_TOKEN * T / (gateup_ms * 1e-3) / 1e12 if gateup_ms > 0 else 0.0
        both_ms = stages["gate_up"] + stages["down"]
        both = EXPERT_FLOP_PER_TOKEN * T / (both_ms * 1e-3) / 1e12 if both_ms > 0 else 0.0
        if world == 1:
            par = "single GPU"
        else:
            par = (f"expert parallel ep{world}, tokens data-parallel, rows exchanged by peer stores over NVLink "
                   f"from inside the expert kernels")
        launches = (KERNELS_PER_PASS + (1 if args.norm else 0)) * n_layers if world == 1 else KERNELS_PER_PASS_EP * n_layers
        line = {
            "metric": METRIC if (T_TOKENS == 4096 and n_layers == 1 and not zipf) else
                      f"MoE-layer prefill tokens/sec at T={T_TOKENS}" + (f" through {n_layers} layers" if n_layers > 1 else ""),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": elapsed_ms / args.steps, "ms_per_step_min": min(regions) / args.steps, "ms_per_step_max": max(regions) / args.steps,
            "regions": len(regions), "higher_is_better": True, "scaling": "strong" if args.strong else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(world, args), "parallelism": par,
                       "l2": "each step streams 1.21 GB of expert weights per layer (> 126 MB L2); no explicit flush",
                       "timing": f"CUDA events on the launching stream around exactly {args.steps} steps, max over ranks; "
                                 f"median of {len(regions)} such regions"},
            "e2e": {"value": tokens * args.steps / e2e_s, "unit": "tokens/s",
                    "h2d_bytes_per_step": T * H * 2 + T * H * 4, "d2h_bytes_per_step": T * H * 4,
                    "regions": len(e2e_regions), "note": "host-buffer call clef_omni_forward_host on layer 0, pinned host memory"},
            "gpu_launches": launches * args.steps,
            "clocks": clock_summary,
            "roofline": {"bound": "tensor", "kernel": "expert_gemm_kernel<gate_up+SwiGLU>", "achieved": achieved,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                         "peak_source": peaks["source"] + " burst cuBLAS bf16 figure; regime of the timed regions: " + regime(clock_summary),
                         "peak_sustained": peaks["bf16_tflops_sustained"], "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                         "traffic": GATEUP_DRAM_TRAFFIC_T4096 if (T == 4096 and world == 1) else None,
                         # gate/up weights once, every token row once (the kernel gathers them), h written once
                         "algorithmic_bytes": (E // world) * 2 * F * H * 2 + T * H * 2 + T * TOP * F * 2},
            "stages_ms": stages,
            "stages_note": f"means per pass from one further region of {args.steps} steps with an event recorded between the stages "
                           f"({marked_ms / args.steps / n_layers:.4f} ms per pass): the marks cost ~20 us per pass and keep a kernel's "
                           f"prologue from overlapping the previous kernel's tail, so the stages sum to more than ms_per_step"
                           + (f" / {n_layers} layers" if n_layers > 1 else ""),
            "expert_gemms": {"tflops": both, "frac_of_bf16_peak": both / peaks["bf16_tflops"],
                             "frac_of_sustained_bf16_peak": both / peaks["bf16_tflops_sustained"]},
            "hbm": {"weights_gbs_over_layer": WEIGHT_BYTES / world / (elapsed_ms / args.steps * per_layer * 1e-3) / 1e9,
                    "peak_gbs": peaks["hbm_gbs"]},
        }
        if ep_equal is not None:
            line["ep_bitwise_equal"] = bool(ep_equal)
        if world == 1 and not args.no_cpu and n_layers == 1 and not zipf:
            r = cpu_reference(T_TOKENS, 3, 1)
            line["cpu_baseline"] = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        b.ep_disconnect()
        dist.barrier()
    b.close()
    if world > 1:
        dist.destroy_process_group()
    if ep_equal is not None and not ep_equal:
        raise SystemExit("expert-parallel output differs from the single-GPU output")


def attention_bench(args):
    """The attention half in front of the block and whole decoder layers (attention half + norm +
    MoE; --layers N stacks them): seeded random weights, text-like positions.  One JSON line with the
    time per pass of the attention half alone and of the layer, and the attention half's FLOP rate
    (projections 2 T (2048 x 5120 + 4096 x 2048), attention 4 x 128 x 32 x sum over records of
    L(L+1)/2).  On N GPUs (weak scaling, T tokens per GPU): the attention half works on the rank's own
    records, the MoE block runs expert-parallel; rank 0 prints the line, every rank checks its bytes
    against a single-GPU context."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from cleffa_b200 import OmniBackend, workloads

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if args.strong:
        raise SystemExit("--attention scales by records (tokens stay with their rank): weak scaling only")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    T, n_layers = T_TOKENS, max(1, args.layers)
    el = E // world
    single = n_layers > 1 or T > 4096
    bounds = np.array([0, T], np.int32) if single else workloads.varlen_bounds(SEED, T)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    peaks = measured_peaks()
    router, gate_up, down = workloads.make_weights(SEED)
    aw = workloads.make_attention_weights(SEED)

    def layer_weights(l):
        """Layer 0: the seeded host weights; further layers from a device generator every rank seeds alike."""
        if l == 0:
            return (router, gate_up, down), (aw["attn_norm"], aw["w_qkv"], aw["w_out"], aw["q_norm"], aw["k_norm"])
        g = torch.Generator(device="cuda").manual_seed(1000 * SEED + l)
        moe = tuple((torch.randn(sh, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                    for sh in ((E, H), (E, 2 * F, H), (E, H, F)))
        qkv, out = [(torch.randn(sh, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16) for sh in ((5120, H), (H, 4096))]
        return moe, (torch.ones(H, device="cuda"), qkv, out, torch.ones(128, device="cuda"), torch.ones(128, device="cuda"))

    def bind(backend, layers, lo, hi):
        for l in range(layers):
            (r_, gu_, dn_), attn = layer_weights(l)
            backend.bind_layer(l, r_.cuda(), gu_[lo:hi].cuda().contiguous(), dn_[lo:hi].cuda().contiguous())
            backend.bind_attention(l, *attn)
            backend.bind_norm(l, torch.ones(H), 1e-6)

    with OmniBackend(local, stream=stream.cuda_stream) as b:
        b.reserve(T, n_layer=n_layers)
        for kv in args.option:
            name, _, val = kv.partition("=")
            b.set_option(name, int(val))
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, b.ep_export())
            b.ep_connect(rank, world, b"".join(handles))
        bind(b, n_layers, rank * el, (rank + 1) * el)
        if world > 1:
            dist.barrier()
            b.ep_sync(30000)
        pos = torch.from_numpy(np.ascontiguousarray(workloads.make_positions(SEED, bounds).T)).cuda()
        x0 = workloads.make_activations(SEED + 1000 * rank, T).float().cuda()
        x = x0.clone()

        def agree(v, op):
            if world == 1:
                return v
            t = torch.tensor([v], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=op)
            return float(t[0])

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def run(attention_only):
            x.copy_(x0)
            b.begin()
            for l in range(n_layers):
                if attention_only:
                    b.encode_attention(l, x, pos, bounds)
                else:
                    b.encode_layer(l, x, pos, bounds)

        def timed(attention_only):
            for _ in range(max(3, args.warmup)):
                run(attention_only)
            b.complete()
            regions = []
            while True:
                barrier()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(stream)
                for _ in range(args.steps):
                    run(attention_only)
                stop.record(stream)
                barrier()
                b.complete()
                regions.append(agree(start.elapsed_time(stop), dist.ReduceOp.MAX if world > 1 else None))
                enough = sum(regions) >= args.min_time_ms or len(regions) >= args.max_regions
                if agree(1.0 if enough else 0.0, dist.ReduceOp.MAX if world > 1 else None) > 0:
                    break
            return statistics.median(regions) / args.steps, len(regions)

        with ClockSampler(local) as sampler:
            attn_ms, n1 = timed(True)
            layer_ms, n2 = timed(False)

        ep_equal = None
        if world > 1:
            # one untimed, checked pass of layer 0: the same tokens through a single-GPU context with all experts
            out_ep = x0.clone()
            b.begin(); b.encode_layer(0, out_ep, pos, bounds); b.complete()
            solo_stream = torch.cuda.Stream()
            with OmniBackend(local, stream=solo_stream.cuda_stream) as solo:
                solo.reserve(T)
                bind(solo, 1, 0, E)
                out_1 = x0.clone()
                torch.cuda.synchronize()
                solo.begin(); solo.encode_layer(0, out_1, pos, bounds); solo.complete()
            ep_equal = agree(1.0 if torch.equal(out_ep, out_1) else 0.0, dist.ReduceOp.MIN) > 0

        if rank == 0:
            lens = np.diff(bounds).astype(np.float64)
            flop = n_layers * (2.0 * T * (H * 5120 + 4096 * H) + 4.0 * 128 * 32 * float((lens * (lens + 1) / 2).sum()))
            line = {
                "metric": f"decoder-layer prefill tokens/sec at T={T}" + (f" through {n_layers} layers" if n_layers > 1 else ""),
                "value": T * world / (layer_ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
                "ms_per_step": layer_ms, "regions": n2, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic",
                "config": {"workload": f"Clef-Omni decoder layer(s): attention half (32/4 heads of 128, causal per record) + RMSNorm + MoE block, T={T} per GPU, "
                                       f"{len(lens)} record(s), {n_layers} layer(s), bf16 weights N(0,0.02), seed {SEED}",
                           "parallelism": "single GPU" if world == 1 else f"records data-parallel, experts ep{world} (rows exchanged by peer stores from inside the expert kernels)",
                           "timing": f"CUDA events around exactly {args.steps} passes, max over ranks, median of the regions"},
                "attention_half": {"ms_per_pass": attn_ms, "ms_per_layer": attn_ms / n_layers, "tflops": flop / (attn_ms * 1e-3) / 1e12,
                                   "frac_of_bf16_peak": flop / (attn_ms * 1e-3) / 1e12 / peaks["bf16_tflops"], "regions": n1,
                                   "flop": flop},
                "moe_half_ms_per_layer": (layer_ms - attn_ms) / n_layers,
                "clocks": sampler.summary(),
            }
            if ep_equal is not None:
                line["ep_bitwise_equal"] = bool(ep_equal)
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            b.ep_disconnect()
            dist.barrier()
    if world > 1:
        dist.destroy_process_group()
    if ep_equal is not None and not ep_equal:
        raise SystemExit("expert-parallel layer output differs from the single-GPU output")


def sweep(args):
    """BASELINE configuration 5: layer latency and achieved weight-streaming bandwidth at small
    batch sizes (seed 4), one GPU.  One JSON line holding the whole table."""
    import numpy as np
    import torch
    from cleffa_b200 import OmniBackend, workloads

    torch.cuda.set_device(0)
    peaks = measured_peaks()
    router, gate_up, down = workloads.make_weights(4)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    rows = []
    with OmniBackend(0, stream=stream.cuda_stream) as b:
        b.reserve(256)
        b.bind_layer(0, router, gate_up, down)
        for T in args.sweep_tokens:
            xn = workloads.make_activations(4, T).cuda()
            x = torch.zeros(T, H, device="cuda")
            for _ in range(5):
                b.begin(); b.encode_moe(0, xn, x)
            b.complete()
            touched = int((b.read("counts") > 0).sum())
            n = 200
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record(stream)
            for _ in range(n):
                b.begin(); b.encode_moe(0, xn, x)
            stop.record(stream)
            b.complete()
            us = start.elapsed_time(stop) * 1e3 / n
            gbs = 9_437_184 * touched / (us * 1e-6) / 1e9
            rows.append({"tokens": T, "us_per_pass": us, "experts_touched": touched, "weight_gbs": gbs,
                         "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "tokens_per_s": T / (us * 1e-6)})
    print(json.dumps({"metric": "MoE-layer latency by batch size (BASELINE configuration 5)", "unit": "us per pass", "n_gpus": 1,
                      "data": "synthetic", "dtype": "bf16", "hbm_peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                      "note": "weight_gbs = 9,437,184 B x experts touched / time; 200 passes between two CUDA events after 5 warm-up passes; "
                              "every pass streams the touched experts' weights (75 MB .. 1.21 GB), L2 is 126 MB: from T=32 on the "
                              "weights exceed it, below that the figure includes L2 hits",
                      "sweep": rows}))


def main():
    global T_TOKENS, SEED
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU (with --strong: of the whole job); default: the headline 4096")
    ap.add_argument("--strong", action="store_true", help="strong scaling: --tokens is the whole job's and is split evenly over the GPUs")
    ap.add_argument("--bias", default="none", choices=["none", "zipf"], help="zipf: BASELINE configuration 4 (use --tokens 8192, seed 3)")
    ap.add_argument("--seed", type=int, default=None, help="workload seed (default 1; 2 with --layers, 3 with --bias zipf)")
    ap.add_argument("--min-time-ms", type=float, default=1000.0, help="repeat the K-step timed region until this much device time was timed")
    ap.add_argument("--max-regions", type=int, default=400)
    ap.add_argument("--attention", action="store_true", help="time the attention half and whole decoder layers (attention + norm + MoE); with --gpus N: records data-parallel, experts sharded (weak scaling)")
    ap.add_argument("--sweep", action="store_true", help="BASELINE configuration 5: latency table over small batch sizes, one GPU")
    ap.add_argument("--sweep-tokens", type=int, nargs="+", default=[1, 8, 32, 64, 128, 256])
    ap.add_argument("--norm", action="store_true", help="with --layers: each layer normalises the residual stream itself (RMSNorm, unit weights) instead of taking a BF16 copy")
    ap.add_argument("--kernels-only", action="store_true", help="run the warm-up and the timed steps and stop (for profiler captures; one GPU)")
    ap.add_argument("--option", action="append", default=[], help="library option name=value (clef_omni_set_option), repeatable")
    ap.add_argument("--layers", type=int, default=1, help="stack of MoE sublayers with residual adds (BASELINE configuration 3 uses 48 at --tokens 16384)")
    args = ap.parse_args()
    T_TOKENS = args.tokens
    SEED = args.seed if args.seed is not None else (3 if args.bias == "zipf" else 2 if args.layers > 1 else 1)
    if args.attention:
        attention_bench(args)
    elif args.sweep:
        sweep(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        ours(args)


if __name__ == "__main__":
    main()
