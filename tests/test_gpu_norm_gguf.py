"""The steps either side of the block, on the GPU through the C-ABI: the RMSNorm in front of
it (clef.metal:190-204; oracle: ref/omni_fp64.py:31-32) and binding from a converted
checkpoint file (clef.c:194-246)."""
import numpy as np
import pytest
import torch

from cleffa_b200 import OmniError
from gguf_writer import BF16, F32, omni_kv, omni_layers, write_gguf
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu
EPS = 1e-6


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().astype(np.int32) & 0xFFFF


def residual(seed, T):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, 2048, generator=g) * (0.25 + 4.0 * torch.rand(T, 1, generator=g))   # rows of different scale
    w = 1.0 + 0.1 * torch.randn(2048, generator=g)
    return x, w


@pytest.mark.parametrize("T", [1, 333, 2500])
def test_norm_in_front_of_the_block(backend, weights0, T):
    b = backend
    b.bind_layer(0, *weights0)
    x0, w = residual(5 + T, T)
    b.bind_norm(0, w, EPS)
    x = x0.cuda()
    b.begin(); b.encode_norm_moe(0, x); b.complete()
    # 1. the normalised rows against FP64, rounded to BF16: equal except where the FP32 result sits
    #    within rounding distance of a BF16 tie, and then one unit apart
    got = b.read("xnorm", T).astype(np.int32)
    want = bf16_bits(orc.rmsnorm(x0, w, EPS).float())
    diff = np.abs(got - want)
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3, (diff.max(), (diff != 0).mean())
    # 2. the block on those rows: the fused call equals norm rows fed to the plain entry point
    xn = torch.from_numpy(got.astype(np.uint16).view(np.int16)).view(torch.bfloat16).reshape(T, 2048).cuda()
    y = x0.cuda()
    b.begin(); b.encode_moe(0, xn, y); b.complete()
    assert torch.equal(x, y)
    # 3. and the oracle's block on the rows the GPU used
    ids, wts = b.read("ids", T), b.read("weights", T)
    ref = orc.experts(xn.cpu(), ids.astype(np.int64), wts.astype(np.float64), weights0[1], weights0[2], residual=x0)
    assert orc.rel_l2(x.cpu(), ref) < 1e-2


def test_norm_needs_weights_and_valid_arguments(backend):
    x = torch.zeros(4, 2048, device="cuda")
    with pytest.raises(OmniError, match="no norm weights bound"):
        backend.begin(); backend.encode_norm_moe(3, x)
    backend.complete()
    with pytest.raises(OmniError, match="invalid Omni norm binding"):
        backend.bind_norm(0, torch.ones(2048), eps=0.0)


def test_all_zero_rows_stay_finite(bound0):
    b = bound0
    b.bind_norm(0, torch.ones(2048), EPS)
    x = torch.zeros(40, 2048, device="cuda")
    x[::2] = torch.randn(20, 2048, generator=torch.Generator().manual_seed(2)).cuda()
    b.begin(); b.encode_norm_moe(0, x); b.complete()
    assert torch.isfinite(x).all()
    assert (b.read("xnorm", 40)[1::2] == 0).all()


def test_bind_from_checkpoint_file(backend, weights0, tmp_path):
    """One full-size layer written as the converter writes it, bound from the file: same bits as
    binding the tensors directly, norm weights included."""
    x0, w = residual(77, 300)
    path = tmp_path / "layer.gguf"
    write_gguf(path, omni_kv(2048, 768, 128, used=8, n_layer=1, eps=EPS), omni_layers([weights0], [w], 2048, 768, 128))
    b = backend
    b.bind_layer(1, *weights0); b.bind_norm(1, w, EPS)
    want = x0.cuda()
    b.begin(); b.encode_norm_moe(1, want); b.complete()
    b.bind_layer(0, *orc.make_weights(9))                  # something else in layer 0 first
    b.bind_gguf(path, 1)
    got = x0.cuda()
    b.begin(); b.encode_norm_moe(0, got); b.complete()
    assert torch.equal(got, want)
    b.bind_layer(0, *weights0)                             # what the session fixture promises
    # a file with the wrong extents is refused and the binding stays
    bad = tmp_path / "bad.gguf"
    write_gguf(bad, omni_kv(2048, 768, 128, used=8, n_layer=1, eps=EPS),
               {"blk.0.ffn_norm.weight": (F32, w), "blk.0.ffn_router.weight": (BF16, weights0[0][:64].contiguous())})
    with pytest.raises(OmniError, match="missing or invalid tensor blk.0.ffn_router.weight"):
        b.bind_gguf(bad, 1)
