"""Generate the golden vectors under tests/golden/ from the reference's own Python code.

Run once, where a checkout of the reference project (zknpr/cleffa) is available:

    python tests/golden/make_golden.py --reference <path to the checkout>

What is stored (small .npz files, committed):

* route_c1.npz   -- what the reference's `ref/omni_fp64.py: route()` returns on the seeded
                    T=512 configuration (seed 0): ids, weights, the nine largest logits and
                    the 8th-9th margin, plus SHA-256 of the generated input bytes so a
                    different random stream is detected instead of silently compared.
* block_c1.npz   -- the output of the Hugging Face FP32 block that ref/omni.py:125-128
                    executes per layer (`Qwen3OmniMoeThinkerTextSparseMoeBlock`, eager
                    experts, FP32 math on the BF16-rounded weights), on the same inputs:
                    32 sampled rows, column sums over all rows and the router's ids.
* rms_small.npz  -- inputs and output of the reference's `ref/omni_fp64.py: rms()` (the FP64
                    RMSNorm in front of the block) on nine seeded rows, among them tiny, large
                    and all-zero ones.
* route_small.npz-- `route()` of the reference on small random FP64 problems (4 experts
                    top-2 and 16 experts top-4), inputs included.

The GPU box has no reference checkout; the tests only read the .npz files.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import omni_oracle as orc  # noqa: E402


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def load_reference_fp64(ref_root: Path):
    spec = importlib.util.spec_from_file_location("ref_omni_fp64", ref_root / "ref" / "omni_fp64.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def hf_block(router, gate_up, down):
    from transformers.models.qwen3_omni_moe import modeling_qwen3_omni_moe as m
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeTextConfig

    cfg = Qwen3OmniMoeTextConfig(hidden_size=router.shape[1], moe_intermediate_size=gate_up.shape[1] // 2,
                                 num_experts=router.shape[0], num_experts_per_tok=orc.TOP, norm_topk_prob=True)
    cfg._experts_implementation = "eager"
    blk = m.Qwen3OmniMoeThinkerTextSparseMoeBlock(cfg)
    with torch.no_grad():
        blk.gate.weight.copy_(router.float())
        blk.experts.gate_up_proj.copy_(gate_up.float())
        blk.experts.down_proj.copy_(down.float())
    return blk.eval()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ap.add_argument("--only", choices=["rms"], help="regenerate one file only")
    args = ap.parse_args()
    ref = load_reference_fp64(Path(args.reference))
    out_dir = Path(__file__).resolve().parent
    torch.set_num_threads(max(1, torch.get_num_threads()))

    # ---- RMSNorm in front of the block: the reference's own ref/omni_fp64.py `rms`
    from types import SimpleNamespace
    g = torch.Generator().manual_seed(23)
    xr = torch.randn(9, 2048, generator=g, dtype=torch.float64)
    xr[1] *= 1e-4; xr[2] *= 300.0; xr[3, 5:] = 0.0; xr[4] = 0.0        # tiny, large, one-hot-ish and all-zero rows
    wr = 1.0 + 0.1 * torch.randn(2048, generator=g, dtype=torch.float64)
    yr = ref.rms(xr, SimpleNamespace(variance_epsilon=1e-6, weight=wr))
    np.savez_compressed(out_dir / "rms_small.npz", x=xr.numpy(), w=wr.numpy(), eps=np.float64(1e-6), y=yr.numpy())
    print("rms: max |restatement - reference| =", float((orc.rmsnorm(xr, wr, 1e-6) - yr).abs().max()))
    if args.only == "rms":
        return

    # ---- configuration 1: T=512, seed 0
    router, gate_up, down = orc.make_weights(0)
    x = orc.make_activations(0, 512)
    with ref.DoubleOnly():
        logits, weights, ids = ref.route(x.double(), router.double(), orc.TOP)
    ranked = torch.sort(logits, dim=-1, descending=True).values[:, : orc.TOP + 1]
    np.savez_compressed(
        out_dir / "route_c1.npz",
        ids=ids.numpy().astype(np.int16), weights=weights.numpy(), top9=ranked.numpy(),
        margin=(ranked[:, orc.TOP - 1] - ranked[:, orc.TOP]).numpy(),
        logits_rows=logits[:8].numpy(),
        sha_x=sha(x), sha_router=sha(router), sha_gate_up=sha(gate_up), sha_down=sha(down))
    mine = orc.route(x, router)
    print("route c1: ids equal to restatement:", bool((mine[2] == ids).all()),
          "max |w - w_ref| =", float((mine[1] - weights).abs().max()),
          "min margin =", float((ranked[:, 7] - ranked[:, 8]).min()))

    blk = hf_block(router, gate_up, down)
    with torch.inference_mode():
        y = blk(x.float()[None])
        y = y[0] if isinstance(y, tuple) else y
        y = y.reshape(512, -1)
        gate_out = blk.gate(x.float())
    hf_ids = gate_out[-1] if isinstance(gate_out, tuple) else None
    rows = np.arange(0, 512, 16)
    fp64_out = orc.experts(x, mine[2], mine[1], gate_up, down)
    print("block c1: rel L2 (HF FP32 vs FP64 restatement) =", orc.rel_l2(y, fp64_out))
    np.savez_compressed(
        out_dir / "block_c1.npz",
        rows=rows.astype(np.int32), y_rows=y[rows].numpy().astype(np.float32),
        col_sum=y.double().sum(0).numpy(), l2=float(y.double().norm()),
        hf_ids=(hf_ids.numpy().astype(np.int16) if hf_ids is not None else np.zeros((0, 8), np.int16)),
        rel_l2_vs_fp64=orc.rel_l2(y, fp64_out))

    # ---- small FP64 routing problems
    g = torch.Generator().manual_seed(11)
    small = {}
    for name, (t, h, e, k) in dict(a=(64, 8, 4, 2), b=(128, 32, 16, 4)).items():
        xs = torch.randn(t, h, generator=g, dtype=torch.float64)
        ws = torch.randn(e, h, generator=g, dtype=torch.float64)
        with ref.DoubleOnly():
            lg, wt, idx = ref.route(xs, ws, k)
        small.update({f"{name}_x": xs.numpy(), f"{name}_w": ws.numpy(), f"{name}_logits": lg.numpy(),
                      f"{name}_weights": wt.numpy(), f"{name}_ids": idx.numpy().astype(np.int16)})
    np.savez_compressed(out_dir / "route_small.npz", **small)
    print("wrote", sorted(p.name for p in out_dir.glob("*.npz")))


if __name__ == "__main__":
    main()
