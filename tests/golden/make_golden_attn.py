"""Generate tests/golden/attn_small.npz from the reference's own Python code.

    python tests/golden/make_golden_attn.py --reference <path to a checkout of zknpr/cleffa>

Calls `text_attention`, `rotary` and `attention` of the reference's ref/omni_fp64.py (FP64, CPU) on
a small seeded problem (hidden 64, 4 query heads, 2 key/value heads, head width 16, rotary
sections 4/2/2, 37 tokens) and stores inputs and outputs.  tests/test_oracle.py checks that
oracle/omni_attn_oracle.py reproduces them; the GPU box has no reference checkout and only reads
the .npz file.
"""
from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def load_reference_fp64(ref_root: Path):
    spec = importlib.util.spec_from_file_location("ref_omni_fp64", ref_root / "ref" / "omni_fp64.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    ref = load_reference_fp64(Path(args.reference))
    g = torch.Generator().manual_seed(11)
    H, nh, nkv, hd, T = 64, 4, 2, 16, 37
    sections, theta, eps = (4, 2, 2), 1e4, 1e-6

    def lin(n_out, n_in):
        m = torch.nn.Linear(n_in, n_out, bias=False, dtype=torch.float64)
        with torch.no_grad():
            m.weight.copy_(torch.randn(n_out, n_in, generator=g, dtype=torch.float64) * 0.2)
        return m

    def norm(n):
        return SimpleNamespace(weight=1.0 + 0.1 * torch.randn(n, generator=g, dtype=torch.float64), variance_epsilon=eps)

    attn = SimpleNamespace(q_proj=lin(nh * hd, H), k_proj=lin(nkv * hd, H), v_proj=lin(nkv * hd, H), o_proj=lin(H, nh * hd),
                           q_norm=norm(hd), k_norm=norm(hd), head_dim=hd)
    layer = SimpleNamespace(self_attn=attn, input_layernorm=norm(H))
    hidden = torch.randn(T, H, generator=g, dtype=torch.float64)
    pos = torch.arange(T).repeat(3, 1)
    pos[1, 5:20] = 5 + torch.randint(0, 6, (15,), generator=g)
    pos[2, 5:20] = 5 + torch.randint(0, 6, (15,), generator=g)
    with torch.inference_mode():
        cos, sin = ref.rotary(pos, hd, theta, list(sections))
        out = ref.text_attention(layer, hidden, (cos, sin))
    np.savez(ROOT / "tests" / "golden" / "attn_small.npz",
             hidden=hidden.numpy(), positions=pos.numpy().astype(np.int32), cos=cos.numpy(), sin=sin.numpy(), out=out.numpy(),
             w_q=attn.q_proj.weight.detach().numpy(), w_k=attn.k_proj.weight.detach().numpy(), w_v=attn.v_proj.weight.detach().numpy(),
             w_o=attn.o_proj.weight.detach().numpy(), attn_norm=layer.input_layernorm.weight.numpy(),
             q_norm=attn.q_norm.weight.numpy(), k_norm=attn.k_norm.weight.numpy(),
             geometry=np.array([H, nh, nkv, hd, T, *sections], np.int64), theta=np.float64(theta), eps=np.float64(eps))
    print("wrote attn_small.npz", out.shape)


if __name__ == "__main__":
    main()
