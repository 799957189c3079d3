"""Host-side mirror of the reference's tensor surface for the attention path.

`TensorF` follows `bten.TensorF` (src/py_tensor_shim.hh:30-158, bound at
:160-288): a 2-D fp32 strided view `(h, w, stride_h, stride_w, offset)` over
device memory (src/utils/tensor.cuh:41-77), with `shape`, `is_cuda`,
`to_numpy`, `copy_from_numpy`, `transpose`/`T`, `slice`, `__getitem__`,
`__matmul__`, `rope`, plus ONE new entry, `attention_fused`, which is the thin
binding the fused kernel adds next to the existing ones.

`AGTensor` follows `mygrad.engine.AGTensor` (mygrad/engine.py:24-63) for what
the attention layer touches: construction from numpy, `.data`, `.shape`,
`.T`, `@`, `.rope`, `.numpy()`.  The fused path is inference-only, so results
carry `requires_grad=False` and no backward closures.

Device memory is a torch CUDA tensor (storage only); all arithmetic goes to the
CUDA library through the C ABI.  Host tensors (`is_cuda=False`) can be created
and copied, but every operator raises "only GPU implementation available", as
the reference's operators do (src/ops/op_rope.cuh:112-114,
src/ops/op_mm_optimized.cuh:78-80).
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import numpy as np
import torch

from . import _lib


def _stream_ptr() -> int:
    # The reference launches everything on the legacy default stream; torch's
    # current stream is that stream unless the caller changed it.
    return torch.cuda.current_stream().cuda_stream


class TensorF:
    """2-D fp32 strided view, mirror of bten.TensorF."""

    def __init__(self, h: int, w: int, is_cuda: bool = True, *, _base: Optional[torch.Tensor] = None,
                 _stride_h: Optional[int] = None, _stride_w: int = 1, _offset: int = 0):
        self.h, self.w = int(h), int(w)
        self.stride_h = int(w if _stride_h is None else _stride_h)
        self.stride_w = int(_stride_w)
        self.offset = int(_offset)
        self.on_device = bool(is_cuda)
        if _base is None:
            _base = torch.empty(self.h * self.w, dtype=torch.float32, device="cuda" if is_cuda else "cpu")
        self.base = _base   # flat fp32 storage shared by views (the role of Tensor<T>::ref)

    # -- construction helpers ------------------------------------------------
    @classmethod
    def from_torch(cls, t: torch.Tensor) -> "TensorF":
        """Wraps a 2-D fp32 torch tensor (any strides) without copying."""
        assert t.dim() == 2 and t.dtype == torch.float32
        base = torch.as_strided(t, (t.untyped_storage().nbytes() // 4,), (1,), 0)
        return cls(t.shape[0], t.shape[1], t.is_cuda, _base=base, _stride_h=t.stride(0), _stride_w=t.stride(1),
                   _offset=t.storage_offset())

    def torch_view(self) -> torch.Tensor:
        return torch.as_strided(self.base, (self.h, self.w), (self.stride_h, self.stride_w), self.offset)

    # -- bten.TensorF surface --------------------------------------------------
    @property
    def shape(self) -> Tuple[int, int]:
        return (self.h, self.w)

    @property
    def is_cuda(self) -> bool:
        return self.on_device

    def copy_from_numpy(self, arr: np.ndarray) -> None:
        if arr.ndim != 2:
            raise RuntimeError("Expected 2D NumPy array")
        if arr.shape != (self.h, self.w):
            raise RuntimeError("Shape mismatch")
        self.torch_view().copy_(torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)))

    def to_numpy(self) -> np.ndarray:
        return self.torch_view().detach().cpu().numpy().copy()

    def fill(self, value: float) -> None:
        self.torch_view().fill_(value)

    def transpose(self) -> "TensorF":
        return TensorF(self.w, self.h, self.on_device, _base=self.base, _stride_h=self.stride_w,
                       _stride_w=self.stride_h, _offset=self.offset)

    T = property(transpose)

    def slice(self, start_h: int, end_h: int, start_w: int, end_w: int) -> "TensorF":
        if start_h >= end_h or end_h > self.h or start_w >= end_w or end_w > self.w:
            raise RuntimeError(f"Slice index out of range: {start_h}:{end_h},{start_w}:{end_w} for tensor {self!r}")
        return TensorF(end_h - start_h, end_w - start_w, self.on_device, _base=self.base, _stride_h=self.stride_h,
                       _stride_w=self.stride_w, _offset=self.offset + start_h * self.stride_h + start_w * self.stride_w)

    def __getitem__(self, index) -> "TensorF":
        if not isinstance(index, tuple):
            index = (index,)
        if len(index) > 2:
            raise IndexError("Tensor only supports 2D indexing")

        def parse(obj, n):
            if obj is Ellipsis or obj is None:
                return 0, n
            if isinstance(obj, slice):
                start, stop, step = obj.indices(n)
                if step != 1:
                    raise IndexError("Tensor slicing only supports step=1")
                return start, stop
            if isinstance(obj, (int, np.integer)):
                i = int(obj) + (n if obj < 0 else 0)
                if not 0 <= i < n:
                    raise IndexError("Index out of range")
                return i, i + 1
            raise TypeError("Tensor indices must be integers, slices, or None")

        sh = parse(index[0] if len(index) > 0 else Ellipsis, self.h)
        sw = parse(index[1] if len(index) > 1 else Ellipsis, self.w)
        return self.slice(sh[0], sh[1], sw[0], sw[1])

    def __repr__(self) -> str:
        return f"dtype=float32 Tensor({self.h}, {self.w}, on_device={'true' if self.on_device else 'false'})"

    # -- raw pointer for the C ABI ----------------------------------------------
    def _ptr(self) -> int:
        return self.base.data_ptr() + 4 * self.offset

    def _require_device(self, what: str) -> None:
        if not self.on_device:
            raise RuntimeError(f"{what}: only GPU implementation available")

    # -- operators ----------------------------------------------------------------
    def __matmul__(self, other: "TensorF") -> "TensorF":
        """op_mm (src/ops/op_mm.cuh:39-57) -> bn_mm_f32."""
        if self.w != other.h:
            raise RuntimeError(f"a,b,out tensor shape mismatch a:{self!r}, b:{other!r}")
        self._require_device("Matrix multiply")
        other._require_device("Matrix multiply")
        out = TensorF(self.h, other.w, True)
        lib = _lib.load()
        _lib.check(lib.bn_mm_f32(self._ptr(), self.stride_h, self.stride_w, other._ptr(), other.stride_h,
                                 other.stride_w, out._ptr(), out.stride_h, out.stride_w, self.h, self.w, other.w,
                                 _stream_ptr()))
        return out

    def rope(self, position_offset: int = 0, head_dim: int = 64, theta: float = 10000.0) -> "TensorF":
        """op_rope (src/ops/op_rope.cuh:101-126) -> bn_rope_f32."""
        self._require_device("RoPE")
        out = TensorF(self.h, self.w, True)
        lib = _lib.load()
        _lib.check(lib.bn_rope_f32(self._ptr(), self.stride_h, self.stride_w, out._ptr(), out.stride_h, out.stride_w,
                                   self.h, self.w, head_dim, theta, position_offset, _stream_ptr()))
        return out

    def argmax(self) -> "TensorU32":
        """Per-row argmax, shape (h, 1): op_argmax (src/ops/op_reduction.cuh:196-210; TensorF.argmax,
        src/py_tensor_shim.hh:220-224) -> bn_argmax_rows_f32.  Ties keep the first index."""
        self._require_device("argmax")
        out = TensorU32(self.h, 1)
        _lib.check(_lib.load().bn_argmax_rows_f32(self._ptr(), self.stride_h, self.stride_w, out.data.data_ptr(),
                                                  self.h, self.w, _stream_ptr()))
        return out

    def gather_rows(self, ids) -> "TensorF":
        """self[ids[i], :] for every i, on the device -> bn_embedding_gather_f32: the device-side form of
        LLaMAModel.embed (mygrad/llama/llama_model.py:58-78).  ids: uint32 numpy array, TensorU32 or torch int tensor."""
        self._require_device("embed")
        if self.stride_w != 1:
            raise RuntimeError("embed: the table must have contiguous rows")
        if isinstance(ids, TensorU32):
            dev_ids = ids.data.reshape(-1)
        elif isinstance(ids, torch.Tensor):
            dev_ids = ids.to(device=self.base.device, dtype=torch.int32).reshape(-1).contiguous()
        else:
            dev_ids = torch.from_numpy(np.ascontiguousarray(ids, dtype=np.uint32).view(np.int32)).to(self.base.device)
        n = int(dev_ids.numel())
        out = TensorF(n, self.w, True)
        err = torch.zeros(1, dtype=torch.int32, device=self.base.device)
        _lib.check(_lib.load().bn_embedding_gather_f32(self._ptr(), self.stride_h, dev_ids.data_ptr(), out._ptr(),
                                                       out.stride_h, n, self.w, self.h, err.data_ptr(), _stream_ptr()))
        if int(err.item()) != 0:
            raise IndexError("index out of range in embedding gather")
        return out

    def rmsnorm(self, weight: "TensorF", eps: float = 1e-6) -> "TensorF":
        """op_rmsnorm (src/ops/op_rmsnorm.cuh:134-157; TensorF.rmsnorm, src/py_tensor_shim.hh:256-260)
        -> bn_rmsnorm_f32.  weight is (1, hidden)."""
        if weight.h != 1 or weight.w != self.w:
            raise RuntimeError("RMSNorm: weight shape must be (1, hidden_dim)")
        if not self.on_device or not weight.on_device:
            raise RuntimeError("RMSNorm: only GPU implementation available")
        out = TensorF(self.h, self.w, True)
        _lib.check(_lib.load().bn_rmsnorm_f32(self._ptr(), self.stride_h, self.stride_w, weight._ptr(), weight.stride_w,
                                              out._ptr(), out.stride_h, out.stride_w, self.h, self.w, float(eps),
                                              _stream_ptr()))
        return out

    def add_rmsnorm(self, residual: "TensorF", weight: "TensorF", eps: float = 1e-6):
        """(self + residual, rmsnorm(self + residual)) in one launch -> bn_add_rmsnorm_f32: the decoder layer's
        `hidden = residual + hidden; hidden = norm(hidden)` (mygrad/llama/llama_layers.py:279-283), bit-identical to
        the reference's two operators."""
        if residual.h != self.h or residual.w != self.w:
            raise RuntimeError("RMSNorm: input/output shape mismatch")
        if weight.h != 1 or weight.w != self.w:
            raise RuntimeError("RMSNorm: weight shape must be (1, hidden_dim)")
        if not self.on_device or not residual.on_device or not weight.on_device:
            raise RuntimeError("RMSNorm: only GPU implementation available")
        total, out = TensorF(self.h, self.w, True), TensorF(self.h, self.w, True)
        _lib.check(_lib.load().bn_add_rmsnorm_f32(
            self._ptr(), self.stride_h, self.stride_w, residual._ptr(), residual.stride_h, residual.stride_w,
            weight._ptr(), weight.stride_w, total._ptr(), total.stride_h, total.stride_w, out._ptr(), out.stride_h,
            out.stride_w, self.h, self.w, float(eps), _stream_ptr()))
        return total, out

    def attention_fused(self, key: "TensorF", value: "TensorF", scale: float, causal: bool = False,
                        seq_offset: int = 0, *, num_heads: int, num_kv_heads: int, head_dim: int,
                        theta: float = 10000.0, heads_mode: int = _lib.BN_HEADS_COLLAPSED,
                        apply_rope: bool = True) -> "TensorF":
        """The new binding entry: self = pre-RoPE query (S, Hq*D); key/value
        (S, Hkv*D).  Argument meaning follows op_attention_fused
        (src/ops/op_attention_fused.cuh:109-118: Q, K, V, out, scale, causal,
        seq_offset) -> bn_attn_prefill_f32."""
        if self.h != key.h or self.h != value.h:
            raise RuntimeError("Attention: batch size mismatch")
        if key.w != value.w or self.w != num_heads * head_dim or key.w != num_kv_heads * head_dim:
            raise RuntimeError("Attention: hidden size mismatch")
        for t in (self, key, value):
            t._require_device("Attention")
        out = TensorF(self.h, self.w, True)
        lib = _lib.load()
        _lib.check(lib.bn_attn_prefill_f32(self._ptr(), self.stride_h, self.stride_w, key._ptr(), key.stride_h,
                                           key.stride_w, value._ptr(), value.stride_h, value.stride_w, out._ptr(),
                                           out.stride_h, out.stride_w, self.h, num_heads, num_kv_heads, head_dim,
                                           float(scale), float(theta), int(seq_offset), int(bool(causal)),
                                           int(heads_mode), int(bool(apply_rope)), _stream_ptr()))
        return out


class TensorU32:
    """Dense (h, w) uint32 tensor on the device (bten.TensorU32): what argmax returns."""

    def __init__(self, h: int, w: int):
        self.h, self.w = int(h), int(w)
        self.data = torch.zeros((self.h, self.w), dtype=torch.int32, device="cuda")   # same bits as uint32
        self.on_device = True

    @property
    def shape(self) -> Tuple[int, int]:
        return (self.h, self.w)

    def to_numpy(self) -> np.ndarray:
        return self.data.cpu().numpy().view(np.uint32).copy()


class AGTensor:
    """Mirror of mygrad.engine.AGTensor for the (inference-only) attention path."""

    def __init__(self, data: Union[np.ndarray, TensorF], children=(), op: str = "", requires_grad: bool = True,
                 is_cuda: Optional[bool] = None):
        self.requires_grad = requires_grad
        self._prev = set(children)
        self._op = op
        self._backward = lambda: None
        self.grad = None
        if isinstance(data, np.ndarray):
            use_cuda = True if is_cuda is None else is_cuda
            t = TensorF(data.shape[0], data.shape[1], use_cuda)
            t.copy_from_numpy(data.astype(np.float32))
            self.data = t
        else:
            self.data = data

    @property
    def shape(self):
        return self.data.shape

    @property
    def is_cuda(self):
        return self.data.is_cuda

    @property
    def T(self) -> "AGTensor":
        return AGTensor(self.data.transpose(), (self,), "T", requires_grad=False)

    def __matmul__(self, other: "AGTensor") -> "AGTensor":
        return AGTensor(self.data @ other.data, (self, other), "@", requires_grad=False)

    def rope(self, position_offset: int = 0, head_dim: int = 64, theta: float = 10000.0) -> "AGTensor":
        return AGTensor(self.data.rope(position_offset, head_dim, theta), (self,), "rope", requires_grad=False)

    def argmax(self):
        """AGTensor.argmax (mygrad/engine.py:355-361): per-row argmax, shape (N, 1), not differentiable."""
        return self.data.argmax()

    def rmsnorm(self, weight: "AGTensor", eps: float = 1e-6) -> "AGTensor":
        """AGTensor.rmsnorm of the reference (forward only here)."""
        return AGTensor(self.data.rmsnorm(weight.data, eps), (self, weight), "rmsnorm", requires_grad=False)

    def add_rmsnorm(self, residual: "AGTensor", weight: "AGTensor", eps: float = 1e-6):
        total, out = self.data.add_rmsnorm(residual.data, weight.data, eps)
        return (AGTensor(total, (self, residual), "+", requires_grad=False),
                AGTensor(out, (self, residual, weight), "add_rmsnorm", requires_grad=False))

    def numpy(self) -> np.ndarray:
        return self.data.to_numpy()

    def __repr__(self) -> str:
        return f"AGTensor(shape={self.shape}, {'cuda' if self.is_cuda else 'cpu'}, op={self._op!r})"
