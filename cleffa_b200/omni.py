"""Python mirror of the C-ABI in include/clef_cuda_omni.h.

The methods keep the names and argument meaning of the reference's Omni module
(clef_metal_omni.m: clef_omni_reserve / begin / encode_layer / complete / trace_reserve,
clef_gpu_dump_routes) so that tests read like the reference's own.  Device memory comes from
torch tensors; only raw pointers cross into the library.  There is no fallback of any kind:
if the shared library is missing or fails to load, importing the backend raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np
import torch

H, F, E, TOP, CHUNK = 2048, 768, 128, 8, 16384
HOST, DEVICE = 0, 1

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libclef_cuda_omni.so"
_ERRLEN = 512


class OmniError(RuntimeError):
    """A library call returned false; the message is the reference-style err string."""


class _Config(C.Structure):
    _fields_ = [("n_layer", C.c_int), ("H", C.c_int), ("ffn", C.c_int), ("n_expert", C.c_int), ("n_expert_used", C.c_int)]


EXPORTS = [
    "clef_cuda_omni_open", "clef_cuda_omni_close", "clef_omni_reserve", "clef_omni_free", "clef_omni_begin",
    "clef_omni_complete", "clef_omni_keepalive", "clef_omni_trace_reserve", "clef_gpu_dump_routes",
    "clef_omni_bind_layer", "clef_omni_encode_moe", "clef_omni_forward_host", "clef_omni_stage_router",
    "clef_omni_stage_route", "clef_omni_stage_assign", "clef_omni_stage_experts", "clef_omni_read",
    "clef_omni_set_option", "clef_omni_profile", "clef_omni_arena_bytes",
    "clef_omni_ep_export", "clef_omni_ep_connect", "clef_omni_ep_connect_local", "clef_omni_ep_disconnect",
    "clef_omni_assign_noalloc", "clef_omni_ep_sync",
    "clef_omni_bind_norm", "clef_omni_encode_norm_moe", "clef_omni_bind_gguf", "clef_omni_gguf_check",
    "clef_omni_bind_attention", "clef_omni_encode_attention", "clef_omni_encode_layer",
]
NOALLOC_MAX_ROWS = 4096
EP_HANDLES, EP_HANDLE_BYTES = 6, 64


def load_library(path: Path | None = None) -> C.CDLL:
    """Loads the library: `path`, else the file named by CLEF_CUDA_OMNI_LIB, else the in-tree build."""
    import os
    path = Path(path) if path else Path(os.environ.get("CLEF_CUDA_OMNI_LIB") or _LIB_PATH)
    if not path.exists():
        raise OmniError(f"{path} is missing: build it with `python -m cleffa_b200.build` (there is no fallback path)")
    lib = C.CDLL(str(path))
    vp, ci, cz, cc = C.c_void_p, C.c_int, C.c_size_t, C.c_char_p
    sig = {
        "clef_cuda_omni_open": (C.c_bool, [C.POINTER(vp), ci, vp, cc, cz]),
        "clef_cuda_omni_close": (None, [vp]),
        "clef_omni_reserve": (C.c_bool, [vp, C.POINTER(_Config), ci, cc, cz]),
        "clef_omni_free": (None, [vp]),
        "clef_omni_begin": (None, [vp]),
        "clef_omni_complete": (C.c_bool, [vp, cc, cz]),
        "clef_omni_keepalive": (None, [vp]),
        "clef_omni_trace_reserve": (C.c_bool, [vp, ci, ci, ci, C.c_bool, cc, cz]),
        "clef_gpu_dump_routes": (C.c_bool, [vp, cc, cc, cz]),
        "clef_omni_bind_layer": (C.c_bool, [vp, ci, vp, vp, vp, vp, ci, cc, cz]),
        "clef_omni_encode_moe": (C.c_bool, [vp, ci, vp, vp, ci, ci, vp, cc, cz]),
        "clef_omni_forward_host": (C.c_bool, [vp, ci, vp, vp, ci, ci, vp, cc, cz]),
        "clef_omni_stage_router": (C.c_bool, [vp, ci, vp, ci, vp, cc, cz]),
        "clef_omni_stage_route": (C.c_bool, [vp, vp, vp, ci, vp, vp, cc, cz]),
        "clef_omni_stage_assign": (C.c_bool, [vp, vp, ci, vp, vp, vp, vp, cc, cz]),
        "clef_omni_stage_experts": (C.c_bool, [vp, ci, vp, vp, vp, vp, ci, cc, cz]),
        "clef_omni_read": (C.c_bool, [vp, cc, vp, cz, cc, cz]),
        "clef_omni_set_option": (C.c_bool, [vp, cc, C.c_long]),
        "clef_omni_profile": (C.c_bool, [vp, C.POINTER(C.c_float)]),
        "clef_omni_arena_bytes": (cz, [vp]),
        "clef_omni_ep_export": (C.c_bool, [vp, vp, cc, cz]),
        "clef_omni_ep_connect": (C.c_bool, [vp, ci, ci, vp, cc, cz]),
        "clef_omni_ep_connect_local": (C.c_bool, [vp, ci, ci, C.POINTER(vp), cc, cz]),
        "clef_omni_ep_disconnect": (None, [vp]),
        "clef_omni_ep_sync": (C.c_bool, [vp, ci, cc, cz]),
        "clef_omni_assign_noalloc": (C.c_bool, [vp, ci, vp, vp, vp, vp, vp, vp, cc, cz]),
        "clef_omni_bind_norm": (C.c_bool, [vp, ci, vp, C.c_float, ci, cc, cz]),
        "clef_omni_encode_norm_moe": (C.c_bool, [vp, ci, vp, ci, ci, vp, cc, cz]),
        "clef_omni_bind_gguf": (C.c_bool, [vp, cc, ci, cc, cz]),
        "clef_omni_bind_attention": (C.c_bool, [vp, ci, vp, vp, vp, vp, vp, C.c_float, C.c_float, ci, cc, cz]),
        "clef_omni_encode_attention": (C.c_bool, [vp, ci, vp, vp, ci, ci, vp, cc, cz]),
        "clef_omni_encode_layer": (C.c_bool, [vp, ci, vp, vp, ci, ci, vp, cc, cz]),
        "clef_omni_gguf_check": (C.c_bool, [cc, ci, ci, ci, ci, C.POINTER(C.c_float), cc, cz]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        if not t.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return C.c_void_p(t.data_ptr())
    if isinstance(t, np.ndarray):
        if not t.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be contiguous")
        return C.c_void_p(t.ctypes.data)
    raise TypeError(type(t))


def assign_noalloc(ids: torch.Tensor, counts, offsets, rowmap, slots, status=None, stream: int | None = None, lib=None):
    """clef_omni_assign_noalloc: the counting sort for callers that must not allocate.  All
    tensors are caller-owned CUDA tensors on the current device; nothing is allocated here or
    in the library.  Raises OmniError with the library's message when the call is refused."""
    lib = lib or load_library()
    err = C.create_string_buffer(_ERRLEN)
    ok = lib.clef_omni_assign_noalloc(_ptr(ids), ids.shape[0], _ptr(counts), _ptr(offsets), _ptr(rowmap), _ptr(slots),
                                      _ptr(status), C.c_void_p(stream) if stream else None, err, _ERRLEN)
    if not ok:
        raise OmniError(err.value.decode())


class OmniBackend:
    """One CUDA context for the Omni MoE block (the `clef_gpu *` of the C-ABI)."""

    def __init__(self, device: int = 0, stream: int | None = None, lib_path: Path | None = None):
        self.lib = load_library(lib_path)
        self.device = device
        self._g = C.c_void_p()
        self._err = C.create_string_buffer(_ERRLEN)
        self._keep = {}
        if not self.lib.clef_cuda_omni_open(C.byref(self._g), device, C.c_void_p(stream) if stream else None, self._err, _ERRLEN):
            raise OmniError(self._err.value.decode())

    # -- helpers
    def _check(self, ok: bool):
        if not ok:
            raise OmniError(self._err.value.decode())

    def close(self):
        if self._g:
            self.lib.clef_cuda_omni_close(self._g)
            self._g = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- reference-named entry points
    def reserve(self, T: int, n_layer: int = 1, H: int = H, ffn: int = F, n_expert: int = E, n_expert_used: int = TOP):
        cfg = _Config(n_layer, H, ffn, n_expert, n_expert_used)
        self._check(self.lib.clef_omni_reserve(self._g, C.byref(cfg), T, self._err, _ERRLEN))

    def free(self):
        self.lib.clef_omni_free(self._g)

    def begin(self):
        self.lib.clef_omni_begin(self._g)

    def complete(self):
        self._check(self.lib.clef_omni_complete(self._g, self._err, _ERRLEN))

    def keepalive(self):
        self.lib.clef_omni_keepalive(self._g)

    def trace_reserve(self, T: int, layers: int, rows: int, enabled: bool = True):
        self._check(self.lib.clef_omni_trace_reserve(self._g, T, layers, rows, enabled, self._err, _ERRLEN))

    def dump_routes(self, path):
        self._check(self.lib.clef_gpu_dump_routes(self._g, str(path).encode(), self._err, _ERRLEN))

    def bind_layer(self, layer: int, router, gate_up, down, bias=None, where: int | None = None):
        """Tensors in the converted layout; host tensors are uploaded, CUDA tensors borrowed
        (and kept alive by this object)."""
        if where is None:
            where = DEVICE if isinstance(router, torch.Tensor) and router.is_cuda else HOST
        n_local = gate_up.shape[0]      # 128, or the rank's slice for device tensors under expert parallelism
        for t, shape in ((router, (E, H)), (gate_up, (n_local, 2 * F, H)), (down, (n_local, H, F))):
            if tuple(t.shape) != shape or t.dtype != torch.bfloat16:
                raise ValueError(f"expected bfloat16 {shape}, got {t.dtype} {tuple(t.shape)}")
        if bias is not None and (tuple(bias.shape) != (E,) or bias.dtype != torch.float32):
            raise ValueError("router bias must be float32 [128]")
        self._check(self.lib.clef_omni_bind_layer(self._g, layer, _ptr(router), _ptr(gate_up), _ptr(down), _ptr(bias),
                                                  where, self._err, _ERRLEN))
        if where == DEVICE:
            self._keep[layer] = (router, gate_up, down, bias)

    def encode_moe(self, layer: int, xn: torch.Tensor, x: torch.Tensor, seq_bounds=None):
        """x[T][2048] (float32, CUDA) += MoE(xn[T][2048] bfloat16, CUDA).  Asynchronous."""
        T = xn.shape[0]
        if xn.dtype != torch.bfloat16 or x.dtype != torch.float32 or tuple(xn.shape) != (T, H) or tuple(x.shape) != (T, H):
            raise ValueError("xn must be bfloat16 [T,2048] and x float32 [T,2048]")
        if seq_bounds is None:
            seq_bounds = np.array([0, T], dtype=np.int32)
        seq_bounds = np.ascontiguousarray(seq_bounds, dtype=np.int32)
        self._check(self.lib.clef_omni_encode_moe(self._g, layer, _ptr(xn), _ptr(x), T, len(seq_bounds) - 1, _ptr(seq_bounds),
                                                  self._err, _ERRLEN))

    def bind_norm(self, layer: int, weight: torch.Tensor, eps: float = 1e-6):
        """FP32 [2048] ffn_norm weights of the layer (host or CUDA tensor; the library copies them)."""
        if tuple(weight.shape) != (H,) or weight.dtype != torch.float32:
            raise ValueError("norm weights must be float32 [2048]")
        weight = weight.contiguous()
        self._check(self.lib.clef_omni_bind_norm(self._g, layer, _ptr(weight), float(eps),
                                                 DEVICE if weight.is_cuda else HOST, self._err, _ERRLEN))

    def encode_norm_moe(self, layer: int, x: torch.Tensor, seq_bounds=None):
        """x[T][2048] (float32, CUDA) += MoE(RMSNorm(x)).  Asynchronous."""
        T = x.shape[0]
        if x.dtype != torch.float32 or tuple(x.shape) != (T, H) or not x.is_cuda:
            raise ValueError("x must be a CUDA float32 [T,2048] tensor")
        if seq_bounds is None:
            seq_bounds = np.array([0, T], dtype=np.int32)
        seq_bounds = np.ascontiguousarray(seq_bounds, dtype=np.int32)
        self._check(self.lib.clef_omni_encode_norm_moe(self._g, layer, _ptr(x), T, len(seq_bounds) - 1, _ptr(seq_bounds),
                                                       self._err, _ERRLEN))

    def bind_attention(self, layer: int, attn_norm, attn_qkv, attn_output, q_norm, k_norm, eps: float = 1e-6, rope_theta: float = 1e6):
        """Tensors of the layer's attention half (host or CUDA tensors, all on the same side; the library copies them)."""
        for t, shape, dt in ((attn_norm, (H,), torch.float32), (attn_qkv, (5120, H), torch.bfloat16), (attn_output, (H, 4096), torch.bfloat16),
                             (q_norm, (128,), torch.float32), (k_norm, (128,), torch.float32)):
            if tuple(t.shape) != shape or t.dtype != dt or not t.is_contiguous():
                raise ValueError(f"expected contiguous {dt} {shape}, got {t.dtype} {tuple(t.shape)}")
        where = DEVICE if attn_qkv.is_cuda else HOST
        self._check(self.lib.clef_omni_bind_attention(self._g, layer, _ptr(attn_norm), _ptr(attn_qkv), _ptr(attn_output), _ptr(q_norm),
                                                      _ptr(k_norm), float(eps), float(rope_theta), where, self._err, _ERRLEN))

    def encode_attention(self, layer: int, x: torch.Tensor, pos3: torch.Tensor, seq_bounds=None):
        """x[T][2048] (float32, CUDA) += attention half; pos3 int32 CUDA [T][3].  Asynchronous."""
        T = x.shape[0]
        if x.dtype != torch.float32 or tuple(x.shape) != (T, H) or not x.is_cuda:
            raise ValueError("x must be a CUDA float32 [T,2048] tensor")
        if pos3.dtype != torch.int32 or tuple(pos3.shape) != (T, 3) or not pos3.is_cuda or not pos3.is_contiguous():
            raise ValueError("pos3 must be a contiguous CUDA int32 [T,3] tensor")
        if seq_bounds is None:
            seq_bounds = np.array([0, T], dtype=np.int32)
        seq_bounds = np.ascontiguousarray(seq_bounds, dtype=np.int32)
        self._check(self.lib.clef_omni_encode_attention(self._g, layer, _ptr(x), _ptr(pos3), T, len(seq_bounds) - 1, _ptr(seq_bounds),
                                                        self._err, _ERRLEN))

    def encode_layer(self, layer: int, x: torch.Tensor, pos3: torch.Tensor, seq_bounds=None):
        """One decoder layer on x[T][2048] (float32, CUDA): attention half, then norm + MoE block."""
        T = x.shape[0]
        if x.dtype != torch.float32 or tuple(x.shape) != (T, H) or not x.is_cuda:
            raise ValueError("x must be a CUDA float32 [T,2048] tensor")
        if pos3.dtype != torch.int32 or tuple(pos3.shape) != (T, 3) or not pos3.is_cuda or not pos3.is_contiguous():
            raise ValueError("pos3 must be a contiguous CUDA int32 [T,3] tensor")
        if seq_bounds is None:
            seq_bounds = np.array([0, T], dtype=np.int32)
        seq_bounds = np.ascontiguousarray(seq_bounds, dtype=np.int32)
        self._check(self.lib.clef_omni_encode_layer(self._g, layer, _ptr(x), _ptr(pos3), T, len(seq_bounds) - 1, _ptr(seq_bounds),
                                                    self._err, _ERRLEN))

    def bind_gguf(self, path, n_layer: int):
        """Bind layers 0..n_layer-1 (experts, router, ffn_norm) from a converted checkpoint file."""
        self._check(self.lib.clef_omni_bind_gguf(self._g, str(path).encode(), n_layer, self._err, _ERRLEN))

    def forward_host(self, layer: int, xn_host: torch.Tensor, x_host: torch.Tensor, seq_bounds=None):
        """Synchronous pass on HOST tensors (x_host is updated in place)."""
        T = xn_host.shape[0]
        if xn_host.is_cuda or x_host.is_cuda or xn_host.dtype != torch.bfloat16 or x_host.dtype != torch.float32:
            raise ValueError("forward_host takes CPU bfloat16 xn and CPU float32 x")
        if seq_bounds is None:
            seq_bounds = np.array([0, T], dtype=np.int32)
        seq_bounds = np.ascontiguousarray(seq_bounds, dtype=np.int32)
        self._check(self.lib.clef_omni_forward_host(self._g, layer, _ptr(xn_host), _ptr(x_host), T, len(seq_bounds) - 1,
                                                    _ptr(seq_bounds), self._err, _ERRLEN))

    # -- stage entry points
    def stage_router(self, layer: int, xn: torch.Tensor) -> torch.Tensor:
        out = torch.empty(xn.shape[0], E, dtype=torch.float64, device=xn.device)
        self._check(self.lib.clef_omni_stage_router(self._g, layer, _ptr(xn), xn.shape[0], _ptr(out), self._err, _ERRLEN))
        return out

    def stage_route(self, hi: torch.Tensor, lo: torch.Tensor | None = None):
        rows = hi.shape[0]
        ids = torch.empty(rows, TOP, dtype=torch.int32, device=hi.device)
        w = torch.empty(rows, TOP, dtype=torch.float32, device=hi.device)
        self._check(self.lib.clef_omni_stage_route(self._g, _ptr(hi), _ptr(lo), rows, _ptr(ids), _ptr(w), self._err, _ERRLEN))
        return ids, w

    def stage_assign(self, ids: torch.Tensor, counts=None, offsets=None, rowmap=None, slots=None):
        rows = ids.shape[0]
        dev = ids.device
        counts = counts if counts is not None else torch.empty(E, dtype=torch.int32, device=dev)
        offsets = offsets if offsets is not None else torch.empty(E + 1, dtype=torch.int32, device=dev)
        rowmap = rowmap if rowmap is not None else torch.empty(rows * TOP, dtype=torch.int32, device=dev)
        slots = slots if slots is not None else torch.empty(rows * TOP, dtype=torch.int32, device=dev)
        self._check(self.lib.clef_omni_stage_assign(self._g, _ptr(ids), rows, _ptr(counts), _ptr(offsets), _ptr(rowmap),
                                                    _ptr(slots), self._err, _ERRLEN))
        return counts, offsets, rowmap, slots

    def stage_experts(self, layer: int, xn, ids, weights, x):
        self._check(self.lib.clef_omni_stage_experts(self._g, layer, _ptr(xn), _ptr(ids), _ptr(weights), _ptr(x),
                                                     xn.shape[0], self._err, _ERRLEN))

    # -- introspection
    _READ = dict(ids=(np.int32, TOP), weights=(np.float32, TOP), logits=(np.float32, E), rowmap=(np.int32, TOP),
                 slots=(np.int32, TOP))

    def read(self, what: str, T: int | None = None) -> np.ndarray:
        if what in self._READ:
            dt, per = self._READ[what]
            out = np.empty((T, per) if what in ("ids", "weights", "logits") else (T * per,), dtype=dt)
        elif what == "xnorm":                      # BF16 bit patterns
            out = np.empty((T, H), np.uint16)
        elif what == "counts":
            out = np.empty(E, np.int32)
        elif what == "offsets":
            out = np.empty(E + 1, np.int32)
        else:
            out = np.empty(1, np.uint32 if what == "status" else np.int32)
        self._check(self.lib.clef_omni_read(self._g, what.encode(), _ptr(out), out.nbytes, self._err, _ERRLEN))
        return out

    # -- expert parallelism
    def ep_export(self) -> bytes:
        """This rank's exchange-buffer handles (6 x 64 bytes) for the other ranks."""
        buf = C.create_string_buffer(EP_HANDLES * EP_HANDLE_BYTES)
        self._check(self.lib.clef_omni_ep_export(self._g, buf, self._err, _ERRLEN))
        return buf.raw

    def ep_connect(self, rank: int, world: int, all_handles: bytes):
        """all_handles: the ep_export() bytes of every rank, concatenated in rank order."""
        if len(all_handles) != world * EP_HANDLES * EP_HANDLE_BYTES:
            raise ValueError("need one handle block per rank")
        buf = C.create_string_buffer(all_handles, len(all_handles))
        self._check(self.lib.clef_omni_ep_connect(self._g, rank, world, buf, self._err, _ERRLEN))

    def ep_connect_local(self, rank: int, world: int, backends):
        """Ranks that live in this process: backends[r] is rank r's OmniBackend."""
        arr = (C.c_void_p * world)(*[b._g for b in backends])
        self._check(self.lib.clef_omni_ep_connect_local(self._g, rank, world, arr, self._err, _ERRLEN))

    def ep_sync(self, timeout_ms: int = 20000):
        """Barrier across the ranks (every rank must call it), waited for on the host."""
        self._check(self.lib.clef_omni_ep_sync(self._g, timeout_ms, self._err, _ERRLEN))

    def ep_disconnect(self):
        self.lib.clef_omni_ep_disconnect(self._g)

    def set_option(self, name: str, value: int):
        if not self.lib.clef_omni_set_option(self._g, name.encode(), int(value)):
            raise OmniError(f"unknown or invalid option {name}={value}")

    def profile(self):
        ms = (C.c_float * 6)()
        if not self.lib.clef_omni_profile(self._g, ms):
            raise OmniError("profiling is off")
        return dict(zip(("router", "permute", "gate_up", "down", "combine", "total"), list(ms)))

    def arena_bytes(self) -> int:
        return int(self.lib.clef_omni_arena_bytes(self._g))
