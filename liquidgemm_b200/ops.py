"""``torch.ops.liquidgemm.*`` on B200, plus the Python entry points of liquidgemm/ops.py.

Importing this module loads the C-ABI CUDA library and registers the ten operator schemas of
the reference (csrc/liquid_gemm/torch_bindings.cpp:43-59) under the same ``liquidgemm``
namespace, with fake (meta) kernels so that ``torch.compile`` and CUDA-graph capture work
(reference liquidgemm/ops.py:16-65).  Each CUDA implementation validates its arguments in
Python -- a bad call raises ``RuntimeError`` before anything reaches the GPU -- allocates its
output (and split-K workspace) with torch, and calls one ``extern "C"`` function on the current
stream.  No op synchronises and none falls back to PyTorch arithmetic.

Like the reference, this module is not imported by the package ``__init__``
(reference liquidgemm/ops.py:3-4).
"""

from __future__ import annotations

import os

import ctypes

import torch

from . import _lib
from ._lib import check, lib
from .quant import LiquidQuantWeight
from .pack import pack_nibbles

_OUT_DTYPES = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}
_DTYPE_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
TILE_BYTES = 8704   # one 128x128 weight tile in the blob: 8192 nibble bytes + 512 metadata bytes

# LIQUIDGEMM_SPLITK is read once per process, like the C++ static of the reference
# (csrc/liquid_gemm/w4a8_wgmma.cu:524-527).
try:
    _SPLITK_ENV = max(0, int(os.environ.get("LIQUIDGEMM_SPLITK", "0") or 0))
except ValueError:
    _SPLITK_ENV = 0

# --------------------------------------------------------------------------------------
# schemas (verbatim operator signatures of the reference) and fake kernels
# --------------------------------------------------------------------------------------
_SCHEMAS = {
    "dequant_weight": "(Tensor qweight, Tensor s_u8, Tensor offset_a, int N, int K, int group_size) -> Tensor",
    "w4a8_gemm": "(Tensor X, Tensor qweight, Tensor s_u8, Tensor offset_a, Tensor s1, Tensor ascale, int N, int K, int group_size) -> Tensor",
    "quant_per_token": "(Tensor x) -> Tensor[]",
    "scale_epilogue": "(Tensor acc, Tensor ascale, Tensor s1, int out_dtype) -> Tensor",
    "wgmma_i8_gemm": "(Tensor a, Tensor b) -> Tensor",
    "w4a8_wgmma": "(Tensor x_i8, Tensor packed, Tensor s_u8, Tensor off_a, int N, int K, int group_size) -> Tensor",
    "wgmma_rs_a_coords": "() -> Tensor",
    "w4a8_wgmma_rs": "(Tensor x_i8, Tensor w, Tensor spack, Tensor s_u8, Tensor off_a, int N, int K, int group_size, bool packed) -> Tensor",
    "w4a8_wgmma_rs_fused": "(Tensor x_i8, Tensor w, Tensor s_u8, Tensor off_a, Tensor ascale, Tensor s1, int N, int K, int group_size, int out_dtype) -> Tensor",
    "w4a8_gemv2": "(Tensor x_i8, Tensor gpack, Tensor s_u8, Tensor off_a, Tensor ascale, Tensor s1, int N, int K, int group_size, int out_dtype) -> Tensor",
    # additions of this library (no reference counterpart): INT8 GEMM with the fused scale epilogue, and the
    # fused W4A8 linear with the bias added inside the kernel's epilogue
    "i8_gemm_scaled": "(Tensor a, Tensor b, Tensor a_scale, Tensor b_scale, int out_dtype) -> Tensor",
    "w4a8_linear_bias": "(Tensor x_i8, Tensor w, Tensor ascale, Tensor s1, Tensor? bias, int N, int K, int out_dtype) -> Tensor",
}

_libdef = torch.library.Library("liquidgemm", "DEF")
for _name, _sig in _SCHEMAS.items():
    _libdef.define(_name + _sig)
_impl = torch.library.Library("liquidgemm", "IMPL", "CUDA")


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


def _dev_ctx(t: torch.Tensor):
    return torch.cuda.device(t.device)


@torch.library.register_fake("liquidgemm::dequant_weight")
def _f_dequant(qweight, s_u8, offset_a, N, K, group_size):
    return qweight.new_empty((N, K), dtype=torch.int8)


@torch.library.register_fake("liquidgemm::w4a8_gemm")
def _f_v1(X, qweight, s_u8, offset_a, s1, ascale, N, K, group_size):
    return X.new_empty((X.shape[0], N), dtype=torch.float32)


@torch.library.register_fake("liquidgemm::quant_per_token")
def _f_qpt(x):
    M, K = x.shape
    return [x.new_empty((M, K), dtype=torch.int8), x.new_empty((M,), dtype=torch.float32)]


@torch.library.register_fake("liquidgemm::scale_epilogue")
def _f_epi(acc, ascale, s1, out_dtype):
    return acc.new_empty(acc.shape, dtype=_OUT_DTYPES[int(out_dtype)])


@torch.library.register_fake("liquidgemm::wgmma_i8_gemm")
def _f_i8(a, b):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=torch.int32)


@torch.library.register_fake("liquidgemm::i8_gemm_scaled")
def _f_i8s(a, b, a_scale, b_scale, out_dtype):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=_OUT_DTYPES[int(out_dtype)])


@torch.library.register_fake("liquidgemm::w4a8_linear_bias")
def _f_lb(x_i8, w, ascale, s1, bias, N, K, out_dtype):
    return x_i8.new_empty((x_i8.shape[0], N), dtype=_OUT_DTYPES[int(out_dtype)])


@torch.library.register_fake("liquidgemm::w4a8_wgmma")
def _f_ss(x_i8, packed, s_u8, off_a, N, K, group_size):
    return x_i8.new_empty((x_i8.shape[0], N), dtype=torch.int32)


@torch.library.register_fake("liquidgemm::w4a8_wgmma_rs")
def _f_rs(x_i8, w, spack, s_u8, off_a, N, K, group_size, packed):
    return x_i8.new_empty((x_i8.shape[0], N), dtype=torch.int32)


@torch.library.register_fake("liquidgemm::w4a8_wgmma_rs_fused")
def _f_rsf(x_i8, w, s_u8, off_a, ascale, s1, N, K, group_size, out_dtype):
    return x_i8.new_empty((x_i8.shape[0], N), dtype=_OUT_DTYPES[int(out_dtype)])


@torch.library.register_fake("liquidgemm::w4a8_gemv2")
def _f_gemv(x_i8, gpack, s_u8, off_a, ascale, s1, N, K, group_size, out_dtype):
    return x_i8.new_empty((x_i8.shape[0], N), dtype=_OUT_DTYPES[int(out_dtype)])


# --------------------------------------------------------------------------------------
# CUDA implementations
# --------------------------------------------------------------------------------------

def _u8(t, name):
    _req(t.is_cuda and t.dtype == torch.uint8, f"{name} must be a CUDA uint8 tensor")
    return t.contiguous()


def _f32(t, name):
    _req(t.is_cuda and t.dtype == torch.float32, f"{name} must be a CUDA float32 tensor")
    return t.contiguous()


def _i8(t, name):
    _req(t.is_cuda and t.dtype == torch.int8 and t.dim() == 2, f"{name} must be a 2-D CUDA int8 tensor")
    return t.contiguous()


def _dequant_weight(qweight, s_u8, offset_a, N, K, group_size):
    _req(qweight.is_cuda, "qweight must be CUDA")
    _req(qweight.dtype == torch.uint8, "qweight must be uint8")
    _req(s_u8.dtype == torch.uint8 and offset_a.dtype == torch.uint8, "s_u8/offset_a must be uint8")
    _req(K % 4 == 0, "K must be a multiple of 4")
    _req(group_size > 0 and group_size % 4 == 0 and K % group_size == 0, "K must be a multiple of group_size")
    _req(qweight.numel() == N * K, "qweight must hold N*K codes (one per byte)")
    G = K // group_size
    _req(s_u8.numel() == N * G and offset_a.numel() == N * G, "s_u8/offset_a must be [N, K/group_size]")
    qweight, s_u8, offset_a = qweight.contiguous(), _u8(s_u8, "s_u8"), _u8(offset_a, "offset_a")
    out = torch.empty((N, K), dtype=torch.int8, device=qweight.device)
    with _dev_ctx(qweight):
        check(lib.lq_dequant_weight(_ptr(qweight), _ptr(s_u8), _ptr(offset_a), _ptr(out), N, K, group_size,
                                    _stream()), "dequant_weight")
    return out


def _quant_per_token(x):
    _req(x.is_cuda and x.dim() == 2, "x must be 2D CUDA")
    _req(x.dtype in _DTYPE_CODES, "x must be bfloat16, float16 or float32")
    x = x.contiguous()
    M, K = x.shape
    xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
    ascale = torch.empty((M,), dtype=torch.float32, device=x.device)
    if M:
        with _dev_ctx(x):
            check(lib.lq_quant_per_token(_ptr(x), _DTYPE_CODES[x.dtype], _ptr(xq), _ptr(ascale), M, K, _stream()),
                  "quant_per_token")
    return [xq, ascale]


def _scale_epilogue(acc, ascale, s1, out_dtype):
    _req(acc.is_cuda and acc.dim() == 2 and acc.dtype == torch.int32, "acc must be a 2-D CUDA int32 tensor")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    acc, ascale, s1 = acc.contiguous(), _f32(ascale, "ascale"), _f32(s1, "s1")
    M, N = acc.shape
    _req(ascale.numel() == M and s1.numel() == N, "ascale must be [M] and s1 [N]")
    y = torch.empty((M, N), dtype=_OUT_DTYPES[int(out_dtype)], device=acc.device)
    if M:
        with _dev_ctx(acc):
            check(lib.lq_scale_epilogue(_ptr(acc), _ptr(ascale), _ptr(s1), _ptr(y), int(out_dtype), M, N, _stream()),
                  "scale_epilogue")
    return y


def _gemv2(x_i8, gpack, s_u8, off_a, ascale, s1, N, K, group_size, out_dtype):
    x_i8 = _i8(x_i8, "x_i8")
    _req(gpack.dtype == torch.uint8 and group_size == 64, "gpack must be uint8 and group_size 64")
    _req(K % 128 == 0, "gemv2 requires K % 128 == 0")
    M = x_i8.shape[0]
    _req(M <= 16, "gemv2 is the M<=16 decode path")
    _req(x_i8.shape[1] == K and gpack.numel() == N * K // 2, "x_i8 must be [M,K] and gpack [N,K/2]")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    gpack, s_u8, off_a = _u8(gpack, "gpack"), _u8(s_u8, "s_u8"), _u8(off_a, "off_a")
    ascale, s1 = _f32(ascale, "ascale"), _f32(s1, "s1")
    _req(s_u8.numel() == N * (K // 64) and off_a.numel() == N * (K // 64), "s_u8/off_a must be [N, K/64]")
    _req(ascale.numel() == M and s1.numel() == N, "ascale must be [M] and s1 [N]")
    y = torch.empty((M, N), dtype=_OUT_DTYPES[int(out_dtype)], device=x_i8.device)
    if M == 0:
        return y
    # One kernel family reads the row-major pack: dp4a up to four tokens, warp-level MMA above.  Layers
    # prepared by this package hold the tile blob instead, which the faster kernels read.
    with _dev_ctx(x_i8):
        check(lib.lq_w4a8_gemv(_ptr(x_i8), _ptr(gpack), _ptr(s_u8), _ptr(off_a), _ptr(ascale), _ptr(s1), _ptr(y),
                               int(out_dtype), M, N, K, group_size, _stream()), "w4a8_gemv2")
    return y


def _splitk_for(M, N, K):
    """Scheduling argument for the tensor-core GEMM: 0 (stream-K) unless LIQUIDGEMM_SPLITK applies."""
    return lib.lq_gemm_pick_splitk(M, N, K, _SPLITK_ENV)


# Zero-filled reduction workspaces, one per (device, stream).  The GEMM kernel needs its workspace
# all-zero on entry and leaves it all-zero on exit, so one buffer serves every call on a stream and
# keeps a stable address under CUDA-graph capture.  Outgrown buffers are kept alive because a
# captured graph may still point at them.
_WORKSPACES: dict = {}
_RETIRED: list = []


def _workspace(nbytes: int, device: torch.device):
    if nbytes == 0:
        return None
    key = (device.index, _stream())
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _RETIRED.append(ws)
        ws = torch.zeros((max(nbytes, 1 << 22),), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def poll_status(device=None) -> None:
    """Read (and clear) the device-side status word of ``device`` (default: the current one) after
    synchronising its current stream.  Kernels never hang: a bounded wait that gives up records a site code
    there and the kernel finishes, possibly with partial sums left in the shared reduction workspaces.  When
    the word is set this function therefore clears every cached workspace of the device and raises
    :class:`liquidgemm_b200._lib.LiquidGemmError`; call it wherever a wrong result must not go unnoticed
    (after a benchmark, between serving batches, in tests)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    with torch.cuda.device(dev):
        rc = lib.lq_poll_status(_stream())
        if rc != 0:
            for (d, _), ws in list(_WORKSPACES.items()):
                if d == dev:
                    ws.zero_()
            torch.cuda.synchronize()
        check(rc, "poll_status")


def _gemm_call(fn_name, x_i8, M, N, K, splitk, call):
    """Run one tensor-core GEMM entry point with the workspace its scheduling needs: fresh scratch for
    the decode-tile planes, or the cached zero-filled reduction buffer of the streaming / persistent
    kernels (cleared again if the enqueue fails; a device-side timeout is reported by
    :func:`poll_status`, which clears it too)."""
    S = _splitk_for(M, N, K) if splitk is None else int(splitk)
    nbytes = lib.lq_gemm_workspace_bytes(M, N, K, S)
    kind = lib.lq_gemm_workspace_kind(M, N, K, S)
    with _dev_ctx(x_i8):
        if kind == 1:
            ws = torch.empty((nbytes,), dtype=torch.uint8, device=x_i8.device)
        else:
            ws = _workspace(nbytes, x_i8.device)
        rc = call(S, _ptr(ws) if ws is not None else None, ws.numel() if ws is not None else 0, _stream())
        if rc != 0 and ws is not None and kind == 2:
            ws.zero_()
        check(rc, fn_name)


def _check_blob(w, N, K):
    _req(w.is_cuda and w.dtype == torch.uint8, "w must be a CUDA uint8 tensor")
    need = lib.lq_tile_blob_bytes(N, K)
    _req(need > 0 and w.numel() == need,
         f"w must be the tile blob of repack_rs_weight for N={N}, K={K} ({need} bytes, got {w.numel()})")
    return w.contiguous()


def gemm_i32(x_i8, blob, N, K, splitk=None):
    """Exact int32 accumulators from a tile blob.  ``splitk``: None = automatic (stream-K unless
    LIQUIDGEMM_SPLITK applies), S >= 1 = that split-K factor, -1 = force the persistent stream-K kernel."""
    x_i8 = _i8(x_i8, "x_i8")
    _req(K % 128 == 0 and x_i8.shape[1] == K, "K%128==0 required and x_i8 must be [M,K]")
    blob = _check_blob(blob, N, K)
    M = x_i8.shape[0]
    acc = torch.empty((M, N), dtype=torch.int32, device=x_i8.device)
    if M:
        _gemm_call("w4a8_gemm_i32", x_i8, M, N, K, splitk,
                   lambda S, ws, nb, st: lib.lq_w4a8_gemm_i32(_ptr(x_i8), _ptr(blob), _ptr(acc), M, N, K, S, ws, nb, st))
    return acc


def gemm_fused(x_i8, blob, ascale, s1, N, K, out_dtype, splitk=None):
    """Fused W4A8 linear from a tile blob (``splitk`` as in :func:`gemm_i32`)."""
    x_i8 = _i8(x_i8, "x_i8")
    _req(K % 128 == 0 and x_i8.shape[1] == K, "K%128==0 required and x_i8 must be [M,K]")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    blob = _check_blob(blob, N, K)
    ascale, s1 = _f32(ascale, "ascale"), _f32(s1, "s1")
    M = x_i8.shape[0]
    _req(ascale.numel() == M and s1.numel() == N, "ascale must be [M] and s1 [N]")
    y = torch.empty((M, N), dtype=_OUT_DTYPES[int(out_dtype)], device=x_i8.device)
    if M:
        _gemm_call("w4a8_gemm_fused", x_i8, M, N, K, splitk,
                   lambda S, ws, nb, st: lib.lq_w4a8_gemm_fused(_ptr(x_i8), _ptr(blob), _ptr(ascale), _ptr(s1), _ptr(y),
                                                                int(out_dtype), M, N, K, S, ws, nb, st))
    return y


def linear_bias(x_i8, blob, ascale, s1, bias, N, K, out_dtype):
    """Fused W4A8 linear from a tile blob with the bias added in the kernel's epilogue (``bias`` may be
    None): ``(T)((T)(acc * ascale[m] * s1[n]) + bias[n])``, bit-identical to the operator followed by
    PyTorch's ``y + bias`` (reference liquidgemm/vllm_plugin.py:205-206)."""
    x_i8 = _i8(x_i8, "x_i8")
    _req(K % 128 == 0 and x_i8.shape[1] == K, "K%128==0 required and x_i8 must be [M,K]")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    blob = _check_blob(blob.reshape(-1), N, K)
    ascale, s1 = _f32(ascale, "ascale"), _f32(s1, "s1")
    M = x_i8.shape[0]
    _req(ascale.numel() == M and s1.numel() == N, "ascale must be [M] and s1 [N]")
    if bias is not None:
        _req(bias.is_cuda and bias.dtype == _OUT_DTYPES[int(out_dtype)] and bias.numel() == N,
             "bias must be a CUDA [N] tensor of the output dtype")
        bias = bias.contiguous()
    y = torch.empty((M, N), dtype=_OUT_DTYPES[int(out_dtype)], device=x_i8.device)
    if M:
        _gemm_call("w4a8_linear_bias", x_i8, M, N, K, 0,
                   lambda S, ws, nb, st: lib.lq_w4a8_linear_bias(_ptr(x_i8), _ptr(blob), _ptr(ascale), _ptr(s1),
                                                                 _ptr(bias) if bias is not None else None, _ptr(y),
                                                                 int(out_dtype), M, N, K, ws, nb, st))
    return y


def quantize_weight_cuda(W: torch.Tensor, group_size: int = 64, want_codes: bool = True, want_blob: bool = False):
    """LiquidQuant quantiser as two CUDA kernels (``lq_quantize_weight``): bit-identical to
    :func:`liquidgemm_b200.quant.quantize_weight` and to the reference's CPU result
    (liquidgemm/quant.py:61-100) without its chain of elementwise launches and host reads.
    Returns ``(LiquidQuantWeight, blob)``; ``qweight_u4`` is None without ``want_codes`` and ``blob`` is
    None without ``want_blob``.  Needs K % 128 == 0 and a group size of 64 or 128."""
    _req(W.is_cuda and W.dim() == 2 and W.dtype in _DTYPE_CODES, "W must be a 2-D CUDA tensor of bf16, fp16 or fp32")
    N, K = W.shape
    _req(K % 128 == 0 and group_size in (64, 128), "K % 128 == 0 and group_size 64 or 128 required")
    W = W.detach().contiguous()
    dev = W.device
    G = K // group_size
    s1 = torch.empty((N,), dtype=torch.float32, device=dev)
    s_u8 = torch.empty((N, G), dtype=torch.uint8, device=dev)
    off = torch.empty((N, G), dtype=torch.uint8, device=dev)
    codes = torch.empty((N, K), dtype=torch.uint8, device=dev) if want_codes else None
    blob = torch.empty(((N + 127) // 128, K // 128, TILE_BYTES), dtype=torch.uint8, device=dev) if want_blob else None
    with _dev_ctx(W):
        check(lib.lq_quantize_weight(_ptr(W), _DTYPE_CODES[W.dtype], N, K, group_size, _ptr(s1), _ptr(s_u8), _ptr(off),
                                     _ptr(codes) if want_codes else None, _ptr(blob) if want_blob else None,
                                     _stream()), "quantize_weight")
    return LiquidQuantWeight(codes, s_u8, off, s1, group_size), blob


def gemv_blob(x_i8, blob, ascale, s1, N, K, out_dtype):
    """Decode GEMV (M <= 8) straight from the GEMM's tile blob: the streaming dp4a kernel."""
    x_i8 = _i8(x_i8, "x_i8")
    _req(K % 128 == 0 and x_i8.shape[1] == K, "K%128==0 required and x_i8 must be [M,K]")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    blob = _check_blob(blob, N, K)
    ascale, s1 = _f32(ascale, "ascale"), _f32(s1, "s1")
    M = x_i8.shape[0]
    _req(M <= 8, "gemv_blob is the M <= 8 decode path")
    _req(ascale.numel() == M and s1.numel() == N, "ascale must be [M] and s1 [N]")
    y = torch.empty((M, N), dtype=_OUT_DTYPES[int(out_dtype)], device=x_i8.device)
    if M:
        with _dev_ctx(x_i8):
            ws = _workspace(lib.lq_gemv_blob_workspace_bytes(), x_i8.device)
            rc = lib.lq_w4a8_gemv_blob(_ptr(x_i8), _ptr(blob), _ptr(ascale), _ptr(s1), _ptr(y), int(out_dtype),
                                       M, N, K, _ptr(ws), ws.numel(), _stream())
            if rc != 0:
                ws.zero_()
            check(rc, "gemv_blob")
    return y


def gemm_fused_scatter(x_i8, blob, ascale, s1, out_ptrs, ld_out, col0, N, K, out_dtype, flag_ptrs=None,
                       flag_index=0, wait_ptr=None, wait_value=0):
    """Fused linear (any M) whose [M, N] output block is stored at column ``col0`` of every matrix in
    ``out_ptrs`` (device addresses of row-major [M, ld_out] buffers of the output dtype: this GPU's and
    its peers' full-width outputs).  The epilogue thereby does the all-gather of an N-sharded layer;
    the caller orders the ranks afterwards (e.g. a symmetric-memory barrier on the same stream, once per
    group of linears whose outputs are consumed together), or lets the kernels do it: with ``flag_ptrs``
    (one uint32 flag array per destination rank) every CTA of the launch that writes the outputs adds 1
    to word ``flag_index`` of each array after its last store, and with ``wait_ptr`` the kernel waits for
    ``*wait_ptr >= wait_value`` before it reads the tokens (``wait_value`` = sum over the ranks of
    decode_grid() of the launch that produced them)."""
    x_i8 = _i8(x_i8, "x_i8")
    _req(K % 128 == 0 and x_i8.shape[1] == K, "K%128==0 required and x_i8 must be [M,K]")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    blob = _check_blob(blob, N, K)
    ascale, s1 = _f32(ascale, "ascale"), _f32(s1, "s1")
    M = x_i8.shape[0]
    _req(M >= 1, "gemm_fused_scatter needs at least one token")
    _req(1 <= len(out_ptrs) <= 8 and ld_out >= N and 0 <= col0 <= ld_out - N, "bad destinations")
    arr = (ctypes.c_void_p * len(out_ptrs))(*[int(p) for p in out_ptrs])
    flags = None
    if flag_ptrs is not None:
        _req(len(flag_ptrs) == len(out_ptrs), "one flag array per destination")
        flags = (ctypes.c_void_p * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
    with _dev_ctx(x_i8):
        nbytes = lib.lq_scatter_workspace_bytes(M, N, K)
        kind = lib.lq_scatter_workspace_kind(M, N, K)
        if kind == 1:
            ws = torch.empty((nbytes,), dtype=torch.uint8, device=x_i8.device)   # split-K planes: plain scratch
        else:
            ws = _workspace(nbytes, x_i8.device)
        rc = lib.lq_w4a8_gemm_fused_scatter_sync(_ptr(x_i8), _ptr(blob), _ptr(ascale), _ptr(s1), arr, len(out_ptrs),
                                                 int(ld_out), int(col0), int(out_dtype), M, N, K, flags,
                                                 int(flag_index), wait_ptr, int(wait_value),
                                                 _ptr(ws) if ws is not None else None,
                                                 ws.numel() if ws is not None else 0, _stream())
        if rc != 0 and ws is not None and kind == 2:
            ws.zero_()
        check(rc, "gemm_fused_scatter")


def decode_grid(M, N, K):
    """CTAs of the launch that writes (and signals) the outputs of a fused linear of this shape on the current
    device: what a consumer of the gather-by-stores epilogue has to see arrive from every rank."""
    return lib.lq_decode_grid(int(M), int(N), int(K))


def _repack_device(src, layout, s_u8, off_a, N, K, group_size):
    _req(K % 128 == 0, "K%128==0 required")
    _req(group_size >= 64 and group_size % 64 == 0 and K % group_size == 0, "group_size must be a multiple of 64")
    src, s_u8, off_a = _u8(src, "weights"), _u8(s_u8, "s_u8"), _u8(off_a, "off_a")
    G = K // group_size
    _req(s_u8.numel() == N * G and off_a.numel() == N * G, "s_u8/off_a must be [N, K/group_size]")
    _req(src.numel() == (N * K if layout == 0 else N * K // 2), "weight tensor has the wrong number of bytes")
    blob = torch.empty(((N + 127) // 128, K // 128, TILE_BYTES), dtype=torch.uint8, device=src.device)
    with _dev_ctx(src):
        check(lib.lq_repack_tiles(_ptr(src), layout, _ptr(s_u8), _ptr(off_a), _ptr(blob), N, K, group_size, _stream()),
              "repack_tiles")
    return blob


def _wgmma_rs(x_i8, w, spack, s_u8, off_a, N, K, group_size, packed):
    _req(w.dtype == torch.uint8 and group_size == 64, "w must be uint8 and group_size 64")
    _req(N % 64 == 0 and K % 128 == 0, "N%64==0 and K%128==0 required")
    if not packed:
        # plain pack_nibbles layout: re-tile into scratch first (reference gathers per element,
        # csrc/liquid_gemm/w4a8_wgmma.cu:424-434)
        w = _repack_device(w, 1, s_u8, off_a, N, K, group_size)
    return gemm_i32(x_i8, w.reshape(-1), N, K)


def _wgmma_rs_fused(x_i8, w, s_u8, off_a, ascale, s1, N, K, group_size, out_dtype):
    _req(w.dtype == torch.uint8 and group_size == 64, "w must be uint8 and group_size 64")
    _req(N % 64 == 0 and K % 128 == 0, "N%64==0 and K%128==0 required")
    return gemm_fused(x_i8, w.reshape(-1), ascale, s1, N, K, out_dtype)


def _wgmma_ss(x_i8, packed, s_u8, off_a, N, K, group_size):
    _req(group_size == 64, "group_size must be 64")
    _req(K % 128 == 0, "K must be a multiple of 128")
    blob = _repack_device(packed, 1, s_u8, off_a, N, K, group_size)
    return gemm_i32(x_i8, blob.reshape(-1), N, K)


def _wgmma_i8(a, b):
    a, b = _i8(a, "a"), _i8(b, "b")
    M, K = a.shape
    N = b.shape[0]
    _req(b.shape[1] == K, "K mismatch")
    _req(K % 128 == 0, "K must be a multiple of 128")
    c = torch.empty((M, N), dtype=torch.int32, device=a.device)
    if M:
        with _dev_ctx(a):
            check(lib.lq_i8_gemm_i32(_ptr(a), _ptr(b), _ptr(c), M, N, K, _stream()), "wgmma_i8_gemm")
    return c


def _i8_gemm_scaled(a, b, a_scale, b_scale, out_dtype):
    a, b = _i8(a, "a"), _i8(b, "b")
    M, K = a.shape
    N = b.shape[0]
    _req(b.shape[1] == K and K % 128 == 0, "K mismatch or K not a multiple of 128")
    _req(int(out_dtype) in _OUT_DTYPES, "out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)")
    a_scale, b_scale = _f32(a_scale, "a_scale").reshape(-1), _f32(b_scale, "b_scale").reshape(-1)
    _req(a_scale.numel() == M and b_scale.numel() == N, "a_scale must have M and b_scale N elements")
    y = torch.empty((M, N), dtype=_OUT_DTYPES[int(out_dtype)], device=a.device)
    if M:
        with _dev_ctx(a):
            check(lib.lq_i8_gemm_scaled(_ptr(a), _ptr(b), _ptr(a_scale), _ptr(b_scale), _ptr(y), int(out_dtype), M, N,
                                        K, _stream()), "i8_gemm_scaled")
    return y


def _gemm_v1(X, qweight, s_u8, offset_a, s1, ascale, N, K, group_size):
    _req(X.is_cuda and qweight.is_cuda, "inputs must be CUDA")
    _req(X.dtype == torch.int8, "X must be int8")
    _req(qweight.dtype == torch.uint8, "qweight must be uint8 (nibble-packed)")
    _req(s1.dtype == torch.float32 and ascale.dtype == torch.float32, "s1/ascale must be float32")
    _req(group_size == 64, "v1 requires group_size == 64")
    _req(K % group_size == 0 and K % 2 == 0, "bad K")
    X, qweight = X.contiguous(), qweight.contiguous()
    s_u8, offset_a, s1, ascale = _u8(s_u8, "s_u8"), _u8(offset_a, "offset_a"), s1.contiguous(), ascale.contiguous()
    M = X.shape[0]
    _req(M <= 16 or K % 128 == 0, "M > 16 requires K % 128 == 0")
    y = torch.empty((M, N), dtype=torch.float32, device=X.device)
    if M == 0:
        return y
    nbytes = lib.lq_gemm_v1_workspace_bytes(M, N, K)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=X.device) if nbytes else None
    with _dev_ctx(X):
        check(lib.lq_w4a8_gemm_v1(_ptr(X), _ptr(qweight), _ptr(s_u8), _ptr(offset_a), _ptr(s1), _ptr(ascale), _ptr(y),
                                  M, N, K, group_size, _ptr(ws) if ws is not None else None, nbytes, _stream()),
              "w4a8_gemm")
    return y


def tile_coords() -> torch.Tensor:
    """(row, k) of every code of a 128x128 weight tile in the order dequant thread ``r`` meets them.

    int32 ``[128, 128, 2]``: entry ``[r, e]`` is the coordinate of the e-th value thread ``r``
    writes to tensor memory (e = 32*chunk + 8*word + 4*half + lane).  Thread r always owns row r
    and walks k in increasing order; the reference's op of the same name dumps the Hopper
    register-fragment coordinates instead (csrc/liquid_gemm/w4a8_wgmma.cu:310-331).
    """
    r = torch.arange(128, dtype=torch.int32).view(128, 1).expand(128, 128)
    k = torch.arange(128, dtype=torch.int32).view(1, 128).expand(128, 128)
    return torch.stack([r, k], dim=-1).contiguous()


def _coords():
    t = tile_coords()
    return t.cuda() if torch.cuda.is_available() else t


_impl.impl("dequant_weight", _dequant_weight)
_impl.impl("quant_per_token", _quant_per_token)
_impl.impl("scale_epilogue", _scale_epilogue)
_impl.impl("w4a8_gemv2", _gemv2)
_impl.impl("w4a8_wgmma_rs", _wgmma_rs)
_impl.impl("w4a8_wgmma_rs_fused", _wgmma_rs_fused)
_impl.impl("w4a8_wgmma", _wgmma_ss)
_impl.impl("wgmma_i8_gemm", _wgmma_i8)
_impl.impl("i8_gemm_scaled", _i8_gemm_scaled)
_impl.impl("w4a8_linear_bias", linear_bias)
_impl.impl("w4a8_gemm", _gemm_v1)
_libdef.impl("wgmma_rs_a_coords", _coords, "CompositeExplicitAutograd")


# --------------------------------------------------------------------------------------
# Python entry points (same names as liquidgemm/ops.py)
# --------------------------------------------------------------------------------------

def pack_gemv_interleaved(qw: LiquidQuantWeight) -> torch.Tensor:
    """Row-major ``[N, K/2]`` pack for the GEMV: byte b of octet h is ``w[8h+b] | w[8h+4+b] << 4``
    so that AND / SHR+AND leave four consecutive k in the byte lanes (reference liquidgemm/ops.py:68-75)."""
    codes = qw.qweight_u4
    n, k = codes.shape
    halves = codes.reshape(n, k // 8, 2, 4)
    return (halves[:, :, 0] | (halves[:, :, 1] << 4)).to(torch.uint8).reshape(n, k // 2).contiguous()


def dequant_weight_i8(qw: LiquidQuantWeight) -> torch.Tensor:
    """INT8 weights [N, K] reconstructed on the device (reference liquidgemm/ops.py:78-87)."""
    return torch.ops.liquidgemm.dequant_weight(qw.qweight_u4.cuda(), qw.s_u8.cuda(), qw.offset_a.cuda(),
                                               qw.N, qw.K, qw.group_size)


def repack_rs_weight(qw: LiquidQuantWeight) -> torch.Tensor:
    """Weight prepack for the tensor-core GEMM: uint8 ``[ceil(N/128), K/128, 8704]`` on the GPU.

    Same role as the reference's fragment-order prepack (liquidgemm/ops.py:118-150) with a layout
    made for B200: per 128x128 tile, four 32-k chunks of ``[128 rows][16 bytes]`` (interleaved
    nibbles, so thread r's four shared loads are conflict free and unpack by mask/shift), then
    ``[128 rows][step0, offset0, step1, offset1]``.  One tile is one contiguous bulk copy.
    """
    return _repack_device(qw.qweight_u4.cuda(), 0, qw.s_u8.cuda(), qw.offset_a.cuda(), qw.N, qw.K, qw.group_size)


def build_rs_scale_pack(qw: LiquidQuantWeight) -> torch.Tensor:
    """Per-tile (step, offset) words ``[ceil(N/128), K/128, 128, 4]`` as they sit inside the blob.

    Kept for signature compatibility: the reference built a separate scale pack and then ignored
    it (liquidgemm/ops.py:153-182, csrc/liquid_gemm/w4a8_wgmma.cu:404); here the words already
    travel inside the tile blob, so the GEMM ops ignore this argument too.
    """
    n, k, g = qw.N, qw.K, qw.group_size
    nt, kt = (n + 127) // 128, k // 128
    halves = torch.arange(k // 64, device=qw.s_u8.device) * 64 // g          # group of every 64-k half tile
    s = qw.s_u8[:, halves].view(n, kt, 2)
    a = qw.offset_a[:, halves].view(n, kt, 2)
    words = torch.stack([s[..., 0], a[..., 0], s[..., 1], a[..., 1]], dim=-1)  # [N, KT, 4]
    out = torch.zeros((nt * 128, kt, 4), dtype=torch.uint8, device=words.device)
    out[:, :, 0::2] = 1
    out[:, :, 1::2] = 128
    out[:n] = words
    return out.view(nt, 128, kt, 4).permute(0, 2, 1, 3).contiguous()


def w4a8_linear_unfused(x_i8, ascale, qw: LiquidQuantWeight, out_dtype: torch.dtype = torch.float16):
    """Unfused pipeline: dequant kernel -> plain INT8 tensor-core GEMM -> scale epilogue.

    Returns ``(y, acc)`` like the reference (liquidgemm/ops.py:90-115), which uses cuBLASLt for
    the middle step; here all three steps are kernels of this library.
    """
    w_i8 = dequant_weight_i8(qw)
    acc = torch.ops.liquidgemm.wgmma_i8_gemm(x_i8.cuda().contiguous(), w_i8)
    y = torch.ops.liquidgemm.scale_epilogue(acc, ascale.cuda().contiguous(), qw.s1.cuda(), _DTYPE_CODES[out_dtype])
    return y, acc


def w4a8_gemm_rs(x_i8, ascale, qw: LiquidQuantWeight, rs_packed: torch.Tensor = None,
                 out_dtype: torch.dtype = torch.float16):
    """Tensor-core W4A8 linear, any M: int32 GEMM then the scale epilogue
    (reference liquidgemm/ops.py:185-201)."""
    if rs_packed is None:
        w, packed = pack_nibbles(qw.qweight_u4).cuda().contiguous(), False
    else:
        w, packed = rs_packed.cuda(), True
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(x_i8.cuda().contiguous(), w, qw.s_u8.cuda(), qw.s_u8.cuda(),
                                             qw.offset_a.cuda(), qw.N, qw.K, qw.group_size, packed)
    return torch.ops.liquidgemm.scale_epilogue(acc, ascale.cuda().contiguous(), qw.s1.cuda(), _DTYPE_CODES[out_dtype])


def w4a8_gemm(x_i8, ascale, qw: LiquidQuantWeight, out_dtype: torch.dtype = torch.float16):
    """Fused W4A8 linear from the plain nibble layout, float32 inside, cast on return
    (reference liquidgemm/ops.py:204-215)."""
    packed = pack_nibbles(qw.qweight_u4).cuda().contiguous()
    y = torch.ops.liquidgemm.w4a8_gemm(x_i8.cuda().contiguous(), packed, qw.s_u8.cuda(), qw.offset_a.cuda(),
                                       qw.s1.cuda(), ascale.cuda(), qw.N, qw.K, qw.group_size)
    return y.to(out_dtype)


def w4a8_linear(x: torch.Tensor, qw_dev: dict, out_dtype: torch.dtype = None) -> torch.Tensor:
    """One W4A8 linear exactly as the vLLM method runs it: quantise tokens, then GEMV (M <= 16 and a
    GEMV pack present) or the fused tensor-core GEMM (reference liquidgemm/vllm_plugin.py:183-196).

    ``qw_dev`` holds device tensors ``s1, s_u8, offset_a, N, K`` and ``rs`` (tile blob) and/or ``gp``.
    """
    odt = _DTYPE_CODES[out_dtype or x.dtype]
    x_i8, ascale = torch.ops.liquidgemm.quant_per_token(x)
    if use_gemv(x_i8.shape[0], qw_dev["N"], qw_dev["K"], qw_dev.get("gp") is not None, qw_dev.get("rs") is not None):
        return torch.ops.liquidgemm.w4a8_gemv2(x_i8, qw_dev["gp"], qw_dev["s_u8"], qw_dev["offset_a"], ascale,
                                               qw_dev["s1"], qw_dev["N"], qw_dev["K"], 64, odt)
    return torch.ops.liquidgemm.w4a8_wgmma_rs_fused(x_i8, qw_dev["rs"], qw_dev["s_u8"], qw_dev["offset_a"], ascale,
                                                    qw_dev["s1"], qw_dev["N"], qw_dev["K"], 64, odt)


_HOST_SCRATCH: dict = {}
_HOST_PLANES: dict = {}
_HOST_SIZES: dict = {}


def w4a8_linear_host(x_host: torch.Tensor, qw_dev: dict, y_host: torch.Tensor = None,
                     out_dtype: torch.dtype = None, stream: "torch.cuda.Stream" = None) -> torch.Tensor:
    """The same linear for activations and outputs in HOST memory (pinned for asynchronous copies):
    upload, quantise, linear from the tile blob ``qw_dev["rs"]`` and download are enqueued on ``stream``
    (default: the current stream of the blob's device) by ONE native call.  Returns ``y_host``
    (allocated pinned when not given); the caller synchronises the stream before reading it.
    Independent requests issued round-robin on a few streams overlap their copies with each other's
    kernels; every stream gets its own scratch and reduction workspace.

    The wrapper is on the per-layer critical path of a host-driven decode loop, so it caches what does
    not change between calls (buffer sizes per shape, the scratch per stream) and does no tensor work."""
    if x_host.is_cuda or x_host.dim() != 2 or not x_host.is_contiguous() or x_host.dtype not in _DTYPE_CODES:
        raise RuntimeError("liquidgemm_b200: x_host must be a contiguous CPU [M,K] tensor of bf16, fp16 or fp32")
    M, K = x_host.shape
    N = qw_dev["N"]
    odt = out_dtype or x_host.dtype
    if K != qw_dev["K"] or K % 128:
        raise RuntimeError("liquidgemm_b200: K mismatch or K % 128 != 0")
    if y_host is None:
        y_host = torch.empty((M, N), dtype=odt, pin_memory=True)
    elif y_host.is_cuda or y_host.dtype != odt or y_host.shape[0] != M or y_host.shape[1] != N or \
            not y_host.is_contiguous():
        raise RuntimeError("liquidgemm_b200: y_host must be a contiguous CPU [M,N] tensor of the output dtype")
    if M == 0:
        return y_host
    blob, s1 = qw_dev["rs"], qw_dev["s1"]
    dev = blob.device
    xc, oc = _DTYPE_CODES[x_host.dtype], _DTYPE_CODES[odt]
    sizes = _HOST_SIZES.get((M, N, K, xc, oc))
    if sizes is None:
        sizes = _HOST_SIZES[(M, N, K, xc, oc)] = (lib.lq_linear_host_scratch_bytes(M, N, K, xc, oc),
                                                  lib.lq_gemm_workspace_bytes(M, N, K, 0),
                                                  lib.lq_gemm_workspace_kind(M, N, K, 0))
    need, nws, kind = sizes
    switch = torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        stream = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
        key = (dev.index, stream)
        scratch = _HOST_SCRATCH.get(key)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                _RETIRED.append(scratch)   # kernels already enqueued on `stream` may still use it
            scratch = torch.empty((max(need, 1 << 22),), dtype=torch.uint8, device=dev)
            _HOST_SCRATCH[key] = scratch
        # kind 2: the shared all-zero reduction buffer (kernels leave it zero); kind 1: split-K planes,
        # plain scratch that must NOT be the zero buffer, because nothing cleans it afterwards
        pool = _WORKSPACES if kind == 2 else _HOST_PLANES
        ws = pool.get(key)
        if nws and (ws is None or ws.numel() < nws):
            if ws is not None:
                _RETIRED.append(ws)
            ws = pool[key] = torch.zeros((max(nws, 1 << 22),), dtype=torch.uint8, device=dev)
            torch.cuda.current_stream().synchronize()   # zero-fill (current stream) before use on `stream`
        rc = lib.lq_w4a8_linear_host(x_host.data_ptr(), xc, blob.data_ptr(), s1.data_ptr(), y_host.data_ptr(), oc,
                                     M, N, K, scratch.data_ptr(), scratch.numel(),
                                     ws.data_ptr() if nws else None, ws.numel() if nws else 0, stream)
        if rc != 0:
            if nws and kind == 2:
                ws.zero_()
            check(rc, "w4a8_linear_host")
    finally:
        if switch:
            torch.cuda.set_device(prev)
    return y_host


class HostStepPlan:
    """A fixed set of host-buffer linears (one decode step of a host-driven loop) recorded once and replayed
    with a single call.

    ``requests`` is a list of ``(x_host, layer, y_host)`` as for :func:`w4a8_linear_host`: pinned host
    activations, a layer dict with the tile blob, a pinned host output.  Construction runs every request
    once (which also sizes the per-stream scratch) and then records the same calls -- host-to-device copy,
    token quantiser, linear, device-to-host copy, spread round-robin over ``n_streams`` streams so that the
    copies of one request overlap the kernels of another -- into a CUDA graph.  :meth:`run` replays it: the
    host pays for one launch instead of four to five driver calls per linear, which is what a step of 5-20 us
    kernels is otherwise dominated by.  The buffers are read and written in place on every replay; call
    :meth:`synchronize` before reading the outputs.  Plans built on the same ``stream`` replay in order.  (The reference drives every linear from Python, one
    operator call at a time: liquidgemm/vllm_plugin.py:174-206.)"""

    def __init__(self, requests, n_streams: int = 3, device=None, stream: "torch.cuda.Stream" = None):
        if not requests:
            raise RuntimeError("liquidgemm_b200: HostStepPlan needs at least one request")
        self.requests = list(requests)
        dev = torch.device(device) if device is not None else self.requests[0][1]["rs"].device
        self.device = dev
        with torch.cuda.device(dev):
            # replays are ordered on `stream`: plans that share it run one after the other, like the steps
            # of a decode loop
            self.main = stream if stream is not None else torch.cuda.Stream()
            self.side = [torch.cuda.Stream() for _ in range(max(1, int(n_streams)))]
            # Requests go to the stream with the least work so far, largest first (bytes streamed and copied
            # stand in for time): the chains of copy -> quantise -> linear -> copy then end together.
            cost = [L["N"] * L["K"] // 2 + 3 * x.numel() + 2 * y.numel() * y.element_size() for x, L, y in self.requests]
            load = [0] * len(self.side)
            self.assignment = [0] * len(self.requests)
            for i in sorted(range(len(self.requests)), key=lambda j: -cost[j]):
                k = min(range(len(self.side)), key=lambda q: load[q])
                self.assignment[i] = k
                load[k] += cost[i]
            # eager pass: allocates scratch and workspaces of every stream outside the capture
            for i, (x, L, y) in enumerate(self.requests):
                w4a8_linear_host(x, L, y, stream=self.side[self.assignment[i]])
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.main):
                for st in self.side:
                    st.wait_stream(self.main)
                for i, (x, L, y) in enumerate(self.requests):
                    w4a8_linear_host(x, L, y, stream=self.side[self.assignment[i]])
                for st in self.side:
                    self.main.wait_stream(st)

    def run(self) -> None:
        """Enqueue the whole step (on the plan's own stream)."""
        with torch.cuda.stream(self.main):
            self.graph.replay()

    def synchronize(self) -> None:
        self.main.synchronize()


def use_gemv(M: int, N: int, K: int, have_gp: bool, have_rs: bool) -> bool:
    """Whether the row-major GEMV pack should serve this call.  Measured on B200 the kernels that read
    the tile blob (streaming dp4a GEMV up to four tokens, tensor-core kernel above) are faster for every
    decode shape, so the GEMV pack is only used by a layer that has nothing else.  The reference
    switches to its GEMV at M <= 16 (liquidgemm/vllm_plugin.py:189)."""
    if not have_gp or M > 16:
        return False
    return not have_rs
