"""fp8 (e4m3) weights in two scale layouts.

:class:`Fp8RowWeight`: one fp32 scale per output feature; activations are quantised per token on
the fly (the "FP8-dynamic" format of the checkpoints the reference benchmarks,
tests/benchmarks/benchmark_utils.py:22-89; per-tensor and per-channel weight scales of
arctic_inference/vllm/spec_dec/fp8.py:140-180 are special cases). The K loop then needs no
rescaling, so the tensor cores run the whole product at the fp8 rate and the scales are applied
once in the epilogue. This is what ``quantization="fp8"`` produces unless the block layout is
asked for.

:class:`Fp8Weight`: block-scaled, one fp32 scale per 128 x 128 block.

:class:`Fp8Weight` behaves like the [N, K] matrix it stands for as far as the model code
needs: ``shape``, row slices and column slices on 128 boundaries (the tensor-parallel shard
views of shift parallelism), so ``ops.linear(x, w)`` works with either a bf16 tensor or an
``Fp8Weight``. The layout matches fp8 block-quantised checkpoints (``weight`` +
``weight_scale_inv``; reference: arctic_inference/vllm/spec_dec/fp8.py:140-180).
"""

from __future__ import annotations

import os

import torch

BLOCK = 128
FP8_MAX = 448.0


class Fp8Weight:
    """``shadow`` is an optional expanded bf16 copy of the same matrix. Decode streams the fp8
    codes (half the bytes per step); long prefill is compute bound and multiplies the shadow
    directly instead of expanding the codes on every call. Whether a model keeps shadows is a
    memory decision made once at load time (:func:`quantize_model_fp8`)."""

    __slots__ = ("q", "scale", "shadow")

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, shadow: torch.Tensor = None):
        assert q.dim() == 2 and scale.dim() == 2
        self.q = q            # [N, K] float8_e4m3fn (row stride free)
        self.scale = scale    # [N/128, K/128] fp32 (row stride free)
        self.shadow = shadow  # [N, K] bf16 or None

    @property
    def shape(self):
        return self.q.shape

    @property
    def device(self):
        return self.q.device

    @property
    def is_cuda(self):
        return self.q.is_cuda

    def numel(self):
        return self.q.numel()

    def __getitem__(self, idx) -> "Fp8Weight":
        if isinstance(idx, slice):
            rows, cols = idx, slice(None)
        else:
            rows, cols = idx

        def blk(s: slice, n: int) -> slice:
            a, b, _ = s.indices(n)
            if a % BLOCK or (b % BLOCK and b != n):
                raise ValueError("fp8 weight slices must fall on 128 boundaries")
            return slice(a // BLOCK, (b + BLOCK - 1) // BLOCK)

        N, K = self.q.shape
        return Fp8Weight(self.q[rows, cols], self.scale[blk(rows, N), blk(cols, K)],
                         None if self.shadow is None else self.shadow[rows, cols])

    def make_shadow(self) -> None:
        self.shadow = self.dequantize().contiguous()

    def dequantize(self) -> torch.Tensor:
        N, K = self.q.shape
        s = self.scale.repeat_interleave(BLOCK, 0)[:N].repeat_interleave(BLOCK, 1)[:, :K]
        return (self.q.float() * s).to(torch.bfloat16)


    def requantize_from(self, dense: torch.Tensor) -> None:
        """Overwrite codes and scales in place (addresses captured in CUDA graphs stay valid)."""
        q = quantize_weight_fp8(dense.to(torch.bfloat16))
        self.q.copy_(q.q)
        self.scale.copy_(q.scale)
        if self.shadow is not None:
            self.shadow.copy_(q.dequantize())


class QuantAct:
    """Activation rows quantised per token: ``q`` e4m3 [M, K], ``scale`` fp32 [M]."""

    __slots__ = ("q", "scale")

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        self.q = q
        self.scale = scale

    @property
    def shape(self):
        return self.q.shape

    @property
    def device(self):
        return self.q.device

    @property
    def is_cuda(self):
        return self.q.is_cuda

    def dequantize(self) -> torch.Tensor:
        return (self.q.float() * self.scale[:, None]).to(torch.bfloat16)


TILE_ROWS, TILE_K = 16, 128


def tile_fp8(q2d: torch.Tensor) -> torch.Tensor:
    """[N, K] codes -> [N/16, K/128, 16, 128]: every 16-row x 128-byte piece contiguous."""
    N, K = q2d.shape
    return q2d.view(N // TILE_ROWS, TILE_ROWS, K // TILE_K, TILE_K).permute(0, 2, 1, 3).contiguous()


class Fp8RowWeight(Fp8Weight):
    """e4m3 codes of an [N, K] matrix with one fp32 scale per output feature (row). Row slices
    carry their scales along; column slices (the K shards of row-parallel layers) keep all of
    them.

    Storage of the codes: row-major [N, K] (the default), or "tiled" (N % 16 == 0 and
    K % 128 == 0) [N/16, K/128, 16, 128], in which each 16-row x 128-byte piece is 2 KB of
    consecutive memory (a GEMM stage's weight tile is then a few dozen KB in 2 KB bursts
    instead of hundreds of 128-byte pieces one row stride apart). Measured on the decode GEMMs
    it is no faster than row-major storage, so nothing selects it by default. Shard views of
    tiled storage are slices of the first two dimensions."""

    __slots__ = ("tiled",)

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, tiled: bool = False):
        assert scale.dim() == 1 and q.dim() == (4 if tiled else 2)
        self.q = q
        self.scale = scale
        self.shadow = None
        self.tiled = tiled
        assert scale.shape[0] == self.shape[0]

    @property
    def shape(self):
        if self.tiled:
            return torch.Size((self.q.shape[0] * TILE_ROWS, self.q.shape[1] * TILE_K))
        return self.q.shape

    def numel(self):
        return self.q.numel()

    def __getitem__(self, idx) -> "Fp8RowWeight":
        if isinstance(idx, slice):
            rows, cols = idx, slice(None)
        else:
            rows, cols = idx
        N, K = self.shape
        a, b, _ = rows.indices(N)
        c, d, _ = cols.indices(K)
        if self.tiled:
            if a % TILE_ROWS or b % TILE_ROWS or c % TILE_K or d % TILE_K:
                raise ValueError("slices of a tiled fp8 weight must fall on 16-row / 128-column "
                                 "boundaries")
            return Fp8RowWeight(self.q[a // TILE_ROWS:b // TILE_ROWS, c // TILE_K:d // TILE_K],
                                self.scale[a:b], True)
        if a % 4 or c % 16:
            raise ValueError("fp8 weight slices must start on 16-byte boundaries")
        return Fp8RowWeight(self.q[rows, cols], self.scale[rows])

    def codes(self) -> torch.Tensor:
        """The codes as a row-major [N, K] tensor (a copy when the storage is tiled)."""
        if not self.tiled:
            return self.q
        N, K = self.shape
        return self.q.permute(0, 2, 1, 3).reshape(N, K)

    def make_shadow(self) -> None:
        pass

    def dequantize(self) -> torch.Tensor:
        return (self.codes().float() * self.scale[:, None]).to(torch.bfloat16)

    def requantize_from(self, dense: torch.Tensor) -> None:
        q = quantize_weight_fp8_row(dense.to(torch.bfloat16), tiled=False)
        self.q.copy_(tile_fp8(q.q) if self.tiled else q.q)
        self.scale.copy_(q.scale)


def quantize_weight_fp8_row(w: torch.Tensor, tiled: bool = False) -> Fp8RowWeight:
    """bf16 [N, K] -> e4m3 codes + one scale per row (scale = amax / 448). ``tiled``: storage
    layout of the codes (see :class:`Fp8RowWeight`); row-major unless asked for."""
    N, K = w.shape
    if K % 16:
        raise ValueError("fp8 quantisation needs K to be a multiple of 16, got %d" % K)
    if tiled and (N % TILE_ROWS or K % TILE_K):
        raise ValueError("tiled fp8 storage needs N %% %d == 0 and K %% %d == 0" % (TILE_ROWS, TILE_K))
    wf = w.float()
    scale = wf.abs().amax(dim=1).clamp_min(1e-10) / FP8_MAX
    q = (wf / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    if tiled:
        return Fp8RowWeight(tile_fp8(q.contiguous()), scale.contiguous(), True)
    return Fp8RowWeight(q.contiguous(), scale.contiguous())


def quant_activation_row_ref(x: torch.Tensor) -> QuantAct:
    """Per-token dynamic quantisation (PyTorch restatement of quant_fp8_row_kernel)."""
    xf = x.float()
    scale = xf.abs().amax(-1).clamp_min(1e-10) / FP8_MAX
    q = (xf * (1.0 / scale)[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return QuantAct(q, scale)


def linear_fp8_row_ref(x, w: Fp8RowWeight, bias=None, residual=None, act=None) -> torch.Tensor:
    """fp32 oracle of ab200_linear_fp8_row; ``x`` is a bf16 tensor or a :class:`QuantAct`."""
    xq = x if isinstance(x, QuantAct) else quant_activation_row_ref(x)
    y = (xq.q.float() @ w.codes().float().t()) * xq.scale[:, None] * w.scale[None, :]
    if bias is not None:
        y = y + bias.float()
    if act == "gelu":
        y = torch.nn.functional.gelu(y)
    if residual is not None:
        y = y + residual.float()
    return y.to(torch.bfloat16)


def quantize_weight_fp8(w: torch.Tensor) -> Fp8Weight:
    """bf16 [N, K] -> e4m3 codes + per-block scales (scale = amax / 448)."""
    N, K = w.shape
    if N % BLOCK or K % BLOCK:
        raise ValueError("fp8 block quantisation needs dimensions that are multiples of 128, "
                         "got %s" % (tuple(w.shape),))
    wf = w.float().view(N // BLOCK, BLOCK, K // BLOCK, BLOCK)
    amax = wf.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (wf / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return Fp8Weight(q.view(N, K).contiguous(), scale.contiguous())


SHADOW_MAX_FRACTION = 0.2     # of the device's memory


def model_fp8_weights(model) -> list:
    out = []
    for lw in model.layers:
        if lw is None:
            continue
        for name in ("wqkv", "wo", "wgu", "wdown"):
            w = getattr(lw, name)
            if isinstance(w, Fp8Weight):
                out.append(w)
    if isinstance(getattr(model, "wkv_swiftkv", None), Fp8Weight):
        out.append(model.wkv_swiftkv)
    return out


def quantize_model_fp8(model, prefill_shadow="auto", scheme: str = "channel") -> None:
    """Replace the linear weights of a decoder with fp8 (embeddings, norms and the LM head stay
    in bf16, as in the fp8 checkpoints the reference serves). ``scheme``: "channel" (one scale
    per output feature, activations per token; the default) or "block" (128 x 128 blocks).

    ``prefill_shadow``: True / False / "auto". With "auto" the expanded bf16 copies are kept
    when they take at most SHADOW_MAX_FRACTION of the GPU's memory (an 8B model's 14 GB on a
    180 GB part), otherwise long prefill expands each weight into a shared scratch matrix."""
    if scheme not in ("channel", "block"):
        raise ValueError("fp8 scheme must be 'channel' or 'block'")
    def quant(w):
        if scheme != "channel":
            return quantize_weight_fp8(w)
        # row-major codes: the tiled storage (see Fp8RowWeight) measured no faster, constrains
        # shard boundaries to 16 rows x 128 columns, and the decode GEMM splits a row-major
        # stage into two TMA boxes, which is worth a few per cent
        # (AB200_FP8_TILED=1 selects the tiles where every rank's shards fall on tile boundaries)
        n, k = w.shape
        ways = max(1, int(getattr(model, "n_stored", 1)))
        tiled = (os.environ.get("AB200_FP8_TILED") == "1" and
                 n % (TILE_ROWS * ways) == 0 and k % (TILE_K * ways) == 0)
        return quantize_weight_fp8_row(w, tiled=tiled)

    for lw in model.layers:
        if lw is None:          # another pipeline stage's layer
            continue
        for name in ("wqkv", "wo", "wgu", "wdown"):
            w = getattr(lw, name)
            if isinstance(w, torch.Tensor):
                setattr(lw, name, quant(w))
                del w
    if getattr(model, "wkv_swiftkv", None) is not None and isinstance(model.wkv_swiftkv, torch.Tensor):
        model.wkv_swiftkv = quant(model.wkv_swiftkv)
    model.act_quant = scheme == "channel"
    on_gpu = torch.cuda.is_available() and model.device.type == "cuda"
    if on_gpu:
        torch.cuda.empty_cache()
    ws = [w for w in model_fp8_weights(model) if not isinstance(w, Fp8RowWeight)]
    if prefill_shadow == "auto":
        need = sum(2 * w.numel() for w in ws)
        total = torch.cuda.get_device_properties(model.device).total_memory if on_gpu else 0
        prefill_shadow = on_gpu and need <= SHADOW_MAX_FRACTION * total
    if prefill_shadow:
        for w in ws:
            w.make_shadow()


def quant_activation_ref(x: torch.Tensor):
    """Per-token, per-128-k dynamic quantisation (PyTorch restatement of quant_fp8_kernel).
    Returns (xq float8 [M, K], sx_t fp32 [K/128, M])."""
    M, K = x.shape
    xf = x.float().view(M, K // BLOCK, BLOCK)
    scale = xf.abs().amax(-1).clamp_min(1e-10) / FP8_MAX
    q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(M, K), scale.t().contiguous()


def linear_fp8_ref(x: torch.Tensor, w: Fp8Weight) -> torch.Tensor:
    xq, sx_t = quant_activation_ref(x)
    M, K = x.shape
    xd = xq.float().view(M, K // BLOCK, BLOCK) * sx_t.t().unsqueeze(-1)
    return (xd.view(M, K) @ w.dequantize().float().t()).to(torch.bfloat16)
