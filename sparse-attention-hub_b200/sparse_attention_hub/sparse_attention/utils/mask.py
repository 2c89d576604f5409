"""`Mask`: a weighted set of key positions per attention row.

Public surface and semantics follow the reference's
`sparse_attention_hub/sparse_attention/utils/mask.py` (constructor :24-110,
factories :174-508, converters :510-611, apply / apply-inverse :614-779,
merges :785-1062, density :1064-1077): value 0 means inactive, any other
value is the weight of the position; the forms are dense, indices/ptr/data
(flat int64 `row * n + col`), full and empty.

On top of those this class carries the *bitmap form* that the sm_100a kernels
produce and consume: `uint32 [rows][W]` active bits with optional per-entry
weights in CSR order.  Native maskers build and extend the bitmap on the
device; the dense and index forms are materialised from it by CUDA kernels
only when somebody asks for them (a user masker calling `get_dense_mask()`,
a test calling `get_index_mask()`).  Once the dense tensor has been handed
out it becomes the single source of truth, because callers are allowed to
write into it in place (the reference's own maskers do, e.g.
maskers/fixed/implementations/basic_fixed.py:361-363).
"""

from __future__ import annotations

import warnings
from typing import Literal, Optional, Tuple

import numpy as np
import torch

from ... import _native


def _n_rows(shape: Tuple[int, ...]) -> int:
    return int(np.prod(shape[:-1])) if len(shape) > 1 else 1


def words_per_row(n_cols: int) -> int:
    """Bitmap words per row: ceil(n/32) rounded up to 16 bytes."""
    w = (n_cols + 31) // 32
    return (w + 3) // 4 * 4


class NativeBits:
    """Device bitmap of a mask plus its lazily built CSR companions.

    Band edits (sink, local window: `add_band`) and the clearing of a fresh bitmap are not
    launched one by one: they are noted and applied by a single kernel when the words are first
    needed (`bits`).  Objects made by `share()` see the same storage and the same notes.

    A masker whose per-entry weights the attention kernel can evaluate by itself (MagicPig)
    hands over a `deferred` payload instead of bits and weights: an object with `device` and
    `materialise() -> NativeBits`.  The attention step reads the payload directly; anybody who
    asks for `bits`, `data` or the CSR arrays gets the materialised form, built once.
    """

    __slots__ = ("_bits", "_lazy", "_data", "ptr", "wpre", "rows", "n_cols", "words", "deferred",
                 "_device")

    MAX_BANDS = 6

    def __init__(self, bits: Optional[torch.Tensor], rows: int, n_cols: int,
                 data: Optional[torch.Tensor] = None, zero_pending: bool = False,
                 deferred=None) -> None:
        if bits is None and deferred is None:
            raise ValueError("a bitmap needs its words or a deferred payload")
        self._bits = bits         # int32 tensor holding uint32 words, [rows, W]
        # edits not yet applied to the storage: {"zero": the storage is uninitialised and stands
        # for an empty bitmap, "sq": query rows per (batch, head), "bands": [(lo_base, lo_qstep,
        # hi_base, hi_qstep, value), ...]}
        self._lazy = {"zero": bool(zero_pending), "sq": 1, "bands": []}
        self.rows = rows
        self.n_cols = n_cols
        self.words = bits.shape[-1] if bits is not None else words_per_row(n_cols)
        self._data = data         # [nnz] in mask dtype or None (all ones)
        self.ptr: Optional[torch.Tensor] = None
        self.wpre: Optional[torch.Tensor] = None
        self.deferred = deferred
        self._device = bits.device if bits is not None else torch.device(deferred.device)

    def _materialise(self) -> None:
        """Swap a deferred payload for its bitmap, weights and CSR arrays."""
        if self._bits is not None:
            return
        other = self.deferred.materialise()
        self._bits, self._lazy = other.bits, {"zero": False, "sq": 1, "bands": []}
        self._data, self.ptr, self.wpre = other.data, other.ptr, other.wpre

    @property
    def data(self) -> Optional[torch.Tensor]:
        self._materialise()
        return self._data

    @data.setter
    def data(self, value: Optional[torch.Tensor]) -> None:
        self._data = value

    @classmethod
    def empty(cls, rows: int, n_cols: int, device: torch.device) -> "NativeBits":
        """An all-zero bitmap whose clearing is deferred to the first band flush."""
        words = words_per_row(n_cols)
        return cls(torch.empty((rows, words), dtype=torch.int32, device=device), rows, n_cols,
                   zero_pending=True)

    def share(self) -> "NativeBits":
        """Same storage and pending edits, CSR companions dropped."""
        self._materialise()
        other = NativeBits(self._bits, self.rows, self.n_cols)
        other._lazy = self._lazy
        return other

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def bits(self) -> torch.Tensor:
        self._materialise()
        if self._lazy["zero"] or self._lazy["bands"]:
            self.flush()
        return self._bits

    @bits.setter
    def bits(self, value: torch.Tensor) -> None:
        self._bits = value
        self._lazy = {"zero": False, "sq": 1, "bands": []}
        self.deferred = None

    def add_band(self, seq_len_queries: int, lo_base: int, lo_qstep: int, hi_base: int,
                 hi_qstep: int, value: int) -> None:
        """Note a band edit (meaning of `sah_mask_fill_band`); valid for unit-weight masks."""
        self._materialise()
        lazy = self._lazy
        if lazy["bands"] and (lazy["sq"] != seq_len_queries or len(lazy["bands"]) >= self.MAX_BANDS):
            self.flush()
        lazy["sq"] = seq_len_queries
        lazy["bands"].append((int(lo_base), int(lo_qstep), int(hi_base), int(hi_qstep), int(value)))
        self.ptr = None   # the CSR companions describe the old bits
        self.wpre = None

    def flush(self) -> None:
        """Apply the pending clear and band edits with one launch."""
        lazy = self._lazy
        bands = lazy["bands"]
        if not lazy["zero"] and not bands:
            return
        import ctypes

        lib = _native.load()
        flat = [x for band in bands for x in band]
        arr = (ctypes.c_int64 * max(len(flat), 1))(*flat)
        _native.check(
            lib.sah_mask_fill_bands(self._bits.data_ptr(), self.rows, lazy["sq"], self.n_cols, self.words,
                                    len(bands), arr, int(lazy["zero"]),
                                    _native.stream_of(self._bits.device)), "sah_mask_fill_bands")
        lazy["zero"] = False
        lazy["bands"] = []

    def ensure_scan(self) -> None:
        """Fill ptr (int64 [rows+1]) and wpre (int32 [rows, W])."""
        self._materialise()
        if self.ptr is not None:
            return
        lib = _native.load()
        dev = self._bits.device
        self.ptr = torch.empty(self.rows + 1, dtype=torch.int64, device=dev)
        self.wpre = torch.empty((self.rows, self.words), dtype=torch.int32, device=dev)
        _native.check(
            lib.sah_mask_rowscan(self.bits.data_ptr(), self.rows, self.words,
                                 self.wpre.data_ptr(), self.ptr.data_ptr(),
                                 _native.stream_of(dev)),
            "sah_mask_rowscan",
        )


class Mask:
    """Weighted position set over a tensor of shape (..., n)."""

    def __init__(
        self,
        shape: Tuple[int, ...],
        dtype: torch.dtype,
        device: torch.device,
        mask: Optional[torch.Tensor] = None,
        indices: Optional[torch.Tensor] = None,
        ptr: Optional[torch.Tensor] = None,
        data: Optional[torch.Tensor] = None,
        from_dense_mask: bool = False,
        from_index: bool = False,
        is_full: bool = False,
        is_empty: bool = False,
    ):
        self.shape = tuple(shape) if not isinstance(shape, tuple) else shape
        self.dtype = dtype
        self.device: torch.device = device
        self.from_dense_mask = from_dense_mask
        self.from_index = from_index
        self.is_full = is_full
        self.is_empty = is_empty
        self._dense: Optional[torch.Tensor] = None
        self._native: Optional[NativeBits] = None
        self.indices: Optional[torch.Tensor] = None
        self.ptr: Optional[torch.Tensor] = None
        self.data: Optional[torch.Tensor] = None

        if is_full or is_empty:
            if device is None:
                raise ValueError("device must be specified for full masks" if is_full
                                 else "device must be specified for empty masks")
        elif from_dense_mask and mask is not None:
            self._dense = mask.to(dtype)
            self.device = mask.device
        elif from_index and indices is not None and ptr is not None:
            self.device = indices.device
            self.indices, self.ptr, self.data = indices, ptr, data
        else:
            raise ValueError(
                "Must specify either from_dense_mask with mask, from_index with indices and ptr, "
                "is_full=True, or is_empty=True"
            )

    # ------------------------------------------------------------------ state
    @property
    def mask(self) -> Optional[torch.Tensor]:
        """Dense tensor of a dense-form mask (materialised from the bitmap on demand)."""
        if self._dense is None and self._native is not None and self.from_dense_mask:
            self._materialise_dense()
        return self._dense

    @mask.setter
    def mask(self, value: Optional[torch.Tensor]) -> None:
        self._dense = value
        if value is not None:
            self._native = None

    def _reset_payload(self) -> None:
        self._dense = None
        self._native = None
        self.indices = None
        self.ptr = None
        self.data = None

    def _become(self, other: "Mask") -> None:
        self.is_full, self.is_empty = other.is_full, other.is_empty
        self.from_dense_mask, self.from_index = other.from_dense_mask, other.from_index
        self._dense, self._native = other._dense, other._native
        self.indices, self.ptr, self.data = other.indices, other.ptr, other.data
        self.device = other.device

    def _detect_full_mask(self, only_check_flag: bool = True) -> bool:
        if self.is_full:
            return True
        if self.is_empty or only_check_flag:
            return False
        if self.from_dense_mask:
            return bool(torch.all(self.get_dense_mask() == 1.0).item())
        if self.from_index and self.indices is not None:
            if self.indices.numel() != int(np.prod(self.shape)):
                return False
            return True if self.data is None else bool(torch.all(self.data == 1.0).item())
        return False

    def _detect_empty_mask(self, only_check_flag: bool = True) -> bool:
        if self.is_empty:
            return True
        if self.is_full or only_check_flag:
            return False
        if self.from_dense_mask:
            return bool(torch.all(self.get_dense_mask() == 0.0).item())
        if self.from_index and self.indices is not None:
            return int(self.indices.numel()) == 0
        return False

    def is_full_mask(self) -> bool:
        return self.is_full

    def is_empty_mask(self) -> bool:
        return self.is_empty

    def __repr__(self) -> str:
        return (
            f"Mask(shape={self.shape}, dtype={self.dtype}, from_dense_mask={self.from_dense_mask}, "
            f"from_index={self.from_index}, is_full={self.is_full}, is_empty={self.is_empty})"
        )

    # -------------------------------------------------------------- factories
    @classmethod
    def create_empty_mask(cls, shape, dtype, device) -> "Mask":
        return cls(shape=shape, dtype=dtype, device=device, is_empty=True)

    @classmethod
    def create_full_mask(cls, shape, dtype, device) -> "Mask":
        return cls(shape=shape, dtype=dtype, device=device, is_full=True)

    @classmethod
    def create_mask_from_indices(cls, shape, indices, ptr, data, dtype) -> "Mask":
        expected = _n_rows(shape) + 1
        if ptr.numel() != expected:
            raise ValueError(f"ptr.numel() must be {expected}, got {ptr.numel()}")
        return cls(shape=shape, dtype=dtype, device=indices.device, indices=indices, ptr=ptr,
                   data=data, from_index=True)

    @classmethod
    def create_mask_from_dense_mask(cls, shape, mask, dtype) -> "Mask":
        if tuple(mask.shape) != tuple(shape):
            raise ValueError(f"mask.shape must be {shape}, got {mask.shape}")
        return cls(shape=shape, dtype=dtype, device=mask.device, mask=mask, from_dense_mask=True)

    @classmethod
    def _from_native(cls, shape, dtype, native: NativeBits) -> "Mask":
        """Dense-semantics mask whose payload is a device bitmap (native maskers)."""
        m = cls(shape=shape, dtype=dtype, device=native.device, is_empty=True)
        m.is_empty = False
        m.from_dense_mask = True
        m._native = native
        return m

    @staticmethod
    def _check_row_wise(shape, row_wise_idx, data) -> None:
        if len(shape) < 1:
            raise ValueError("shape must have at least one dimension")
        if row_wise_idx.shape[-1] <= 0:
            raise ValueError("row_wise_idx must have at least one column")
        want = tuple(shape[:-1]) + (row_wise_idx.shape[-1],)
        if tuple(row_wise_idx.shape) != want:
            raise ValueError(f"row_wise_idx.shape must be {want}, got {row_wise_idx.shape}")
        if data.shape != row_wise_idx.shape:
            raise ValueError(
                f"data.shape must match row_wise_idx.shape {row_wise_idx.shape}, got {data.shape}"
            )

    @classmethod
    def create_from_row_wise_idx(cls, shape, row_wise_idx, data,
                                 mask_type: Literal["index", "dense"], dtype,
                                 use_padding: bool = False,
                                 mode: Literal["sparse", "dense"] = "dense") -> "Mask":
        if mode == "sparse":
            if mask_type == "dense":
                warnings.warn(
                    "Creating dense mask in sparse mode is SLOW. Unless you know what you are "
                    "doing, use dense mode instead.", UserWarning, stacklevel=2)
            return cls.create_from_row_wise_idx_sparse(shape, row_wise_idx, data, mask_type,
                                                       dtype, use_padding)
        if mode == "dense":
            if mask_type == "index":
                warnings.warn(
                    "Creating index mask in dense mode is SLOW. Unless you know what you are "
                    "doing, use sparse mode instead.", UserWarning, stacklevel=2)
            return cls.create_from_row_wise_idx_dense(shape, row_wise_idx, data, mask_type,
                                                      dtype, use_padding)
        raise ValueError(f"Invalid mode: {mode}")

    @classmethod
    def create_from_row_wise_idx_dense(cls, shape, row_wise_idx, data, mask_type, dtype,
                                       use_padding: bool = False) -> "Mask":
        cls._check_row_wise(shape, row_wise_idx, data)
        assert not use_padding, "use_padding is not supported for dense mode; use sparse mode instead"
        if mask_type not in ("dense", "index"):
            raise ValueError(f"type must be 'index' or 'dense', got {mask_type}")
        if row_wise_idx.is_cuda and dtype in (torch.float32, torch.bfloat16):
            # deterministic on the device: the last duplicate of a column wins, as on the CPU
            lib = _native.load()
            rows, n, k = _n_rows(shape), shape[-1], row_wise_idx.shape[-1]
            idx = row_wise_idx.to(torch.int64).contiguous()
            vals = data.to(device=idx.device, dtype=dtype).contiguous()
            claims = torch.empty(rows * n, dtype=torch.int64, device=idx.device)
            dense = torch.empty(tuple(shape), dtype=dtype, device=idx.device)
            _native.check(
                lib.sah_mask_rowwise_scatter(idx.data_ptr(), vals.data_ptr(), _native.dtype_code(dtype), rows, k,
                                             n, claims.data_ptr(), dense.data_ptr(),
                                             _native.stream_of(idx.device)), "sah_mask_rowwise_scatter")
            return cls.create_mask_from_dense_mask(shape, dense, dtype=dtype)
        dense = torch.zeros(shape, dtype=dtype, device=row_wise_idx.device)
        dense.scatter_(dim=-1, index=row_wise_idx, src=data.to(dtype))
        return cls.create_mask_from_dense_mask(shape, dense, dtype=dtype)

    @classmethod
    def create_from_row_wise_idx_sparse(cls, shape, row_wise_idx, data, mask_type, dtype,
                                        use_padding: bool = False) -> "Mask":
        cls._check_row_wise(shape, row_wise_idx, data)
        if mask_type not in ("dense", "index"):
            raise ValueError(f"type must be 'index' or 'dense', got {mask_type}")
        n = shape[-1]
        rows = _n_rows(shape)
        k = row_wise_idx.shape[-1]
        dev = row_wise_idx.device
        cols = row_wise_idx.reshape(rows, k)
        vals = data.reshape(rows, k)
        flat = cols + torch.arange(rows, device=dev).unsqueeze(1) * n
        if use_padding:
            keep = cols >= 0
            ptr = torch.zeros(rows + 1, dtype=torch.long, device=dev)
            ptr[1:] = torch.cumsum(keep.sum(dim=1), dim=0)
            flat, vals = flat[keep], vals[keep]
        else:
            ptr = torch.arange(0, rows * k + 1, k, dtype=torch.long, device=dev)
            flat, vals = flat.reshape(-1), vals.reshape(-1)
        sparse = cls.create_mask_from_indices(shape, flat, ptr, vals, dtype=dtype)
        if mask_type == "dense":
            return cls.create_mask_from_dense_mask(shape, sparse.get_dense_mask(), dtype=dtype)
        return sparse

    # ------------------------------------------------------------ conversions
    def _materialise_dense(self) -> None:
        nb = self._native
        assert nb is not None
        lib = _native.load()
        dense = torch.empty(self.shape, dtype=self.dtype, device=nb.bits.device)
        if nb.data is not None:
            nb.ensure_scan()
        _native.check(
            lib.sah_mask_bits_to_dense(
                nb.bits.data_ptr(), _native.ptr(nb.data), _native.ptr(nb.wpre), _native.ptr(nb.ptr),
                _native.dtype_code(self.dtype), nb.rows, nb.n_cols, nb.words, dense.data_ptr(),
                _native.stream_of(nb.bits.device)),
            "sah_mask_bits_to_dense",
        )
        # The dense tensor may now be edited in place by its holder.
        self._dense = dense
        self._native = None

    def get_dense_mask(self) -> torch.Tensor:
        if self.is_full:
            return torch.ones(self.shape, dtype=self.dtype, device=self.device)
        if self.is_empty:
            return torch.zeros(self.shape, dtype=self.dtype, device=self.device)
        if self.from_dense_mask:
            dense = self.mask
            if dense is None:
                raise RuntimeError("Dense mask is None")
            return dense
        if self.from_index:
            if self.indices is None or self.ptr is None:
                raise RuntimeError("Sparse mask indices or ptr is None")
            dense = torch.zeros(self.shape, dtype=self.dtype, device=self.indices.device)
            if len(self.indices) > 0:
                dense.view(-1)[self.indices] = 1.0 if self.data is None else self.data.to(self.dtype)
            return dense
        raise RuntimeError("Mask object is in an invalid state")

    def get_index_mask(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        rows, n = _n_rows(self.shape), self.shape[-1]
        if self.is_full:
            total = int(np.prod(self.shape))
            return (torch.arange(total, dtype=torch.long, device=self.device),
                    torch.arange(0, total + 1, n, dtype=torch.long, device=self.device),
                    torch.ones(total, dtype=self.dtype, device=self.device))
        if self.is_empty:
            return (torch.empty(0, dtype=torch.long, device=self.device),
                    torch.zeros(rows + 1, dtype=torch.long, device=self.device),
                    torch.empty(0, dtype=self.dtype, device=self.device))
        if self.from_index:
            if self.indices is None or self.ptr is None:
                raise RuntimeError("Sparse mask indices or ptr is None")
            data = self.data
            if data is None:
                data = torch.ones(self.indices.numel(), dtype=self.dtype, device=self.indices.device)
            return self.indices, self.ptr, data
        if self.from_dense_mask:
            if self._native is not None or (self._dense is not None and self._dense.is_cuda
                                            and self.dtype in (torch.float32, torch.bfloat16)):
                return self._index_from_native()
            dense = self._dense
            if dense is None:
                raise RuntimeError("Dense mask is None")
            flat = dense.reshape(-1)
            idx = torch.nonzero(flat, as_tuple=False).squeeze(-1)
            ptr = torch.zeros(rows + 1, dtype=torch.long, device=dense.device)
            ptr[1:] = torch.cumsum(torch.count_nonzero(dense.reshape(rows, n), dim=1), dim=0)
            return idx, ptr, flat[idx]
        raise RuntimeError("Mask object is in an invalid state")

    def _index_from_native(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        nb = self.native_bits()
        nb.ensure_scan()
        lib = _native.load()
        dev = nb.bits.device
        nnz = int(nb.ptr[-1].item())
        idx = torch.empty(nnz, dtype=torch.int64, device=dev)
        if nnz > 0:
            _native.check(
                lib.sah_mask_bits_to_indices(nb.bits.data_ptr(), nb.wpre.data_ptr(),
                                             nb.ptr.data_ptr(), nb.rows, nb.n_cols, nb.words,
                                             idx.data_ptr(), _native.stream_of(dev)),
                "sah_mask_bits_to_indices",
            )
        data = nb.data[:nnz] if nb.data is not None else torch.ones(nnz, dtype=self.dtype, device=dev)
        return idx, nb.ptr, data

    def native_bits(self) -> NativeBits:
        """Bitmap form on the device, built by CUDA kernels from whatever form is held.

        Raises NativeLibraryError for masks that do not live on a CUDA device.
        """
        if self._native is not None:
            return self._native
        rows, n = _n_rows(self.shape), self.shape[-1]
        words = words_per_row(n)
        dev = torch.device(self.device)
        if dev.type != "cuda":
            raise _native.NativeLibraryError(
                f"mask lives on {dev}; the native path runs on CUDA devices only and has no "
                "CPU fallback")
        lib = _native.load()
        st = _native.stream_of(dev)
        if self.is_empty:
            return NativeBits.empty(rows, n, dev)
        if self.is_full:
            bits = torch.zeros((rows, words), dtype=torch.int32, device=dev)
            _native.check(lib.sah_mask_fill_band(bits.data_ptr(), rows, 1, n, words, 0, 0, n, 0, 1, st),
                          "sah_mask_fill_band")
            return NativeBits(bits, rows, n)
        dense = self.get_dense_mask().contiguous()
        code = _native.dtype_code(self.dtype)
        bits = torch.empty((rows, words), dtype=torch.int32, device=dev)
        _native.check(lib.sah_mask_dense_to_bits(dense.data_ptr(), code, rows, n, words,
                                                 bits.data_ptr(), st), "sah_mask_dense_to_bits")
        nb = NativeBits(bits, rows, n)
        nb.ensure_scan()
        nnz = int(nb.ptr[-1].item())
        data = torch.empty(nnz, dtype=self.dtype, device=dev)
        if nnz > 0:
            _native.check(
                lib.sah_mask_dense_gather_data(dense.data_ptr(), code, bits.data_ptr(),
                                               nb.wpre.data_ptr(), nb.ptr.data_ptr(), rows, n,
                                               words, data.data_ptr(), st),
                "sah_mask_dense_gather_data")
        nb.data = data
        # Not cached: a dense or index payload may be edited by its holder.
        return nb

    # ------------------------------------------------------------------ apply
    def _check_input(self, x: torch.Tensor) -> None:
        if tuple(x.shape) != tuple(self.shape):
            raise ValueError(f"input_tensor.shape must be {self.shape}, got {x.shape}")

    def apply_mask(self, input_tensor, mode: Literal["sparse", "dense"] = "dense"):
        if mode == "sparse":
            return self.apply_mask_sparse(input_tensor)
        if mode == "dense":
            return self.apply_mask_dense(input_tensor)
        raise ValueError(f"Invalid mode: {mode}")

    def apply_mask_dense(self, input_tensor):
        self._check_input(input_tensor)
        if self.is_full or self.is_empty:
            return input_tensor
        return input_tensor * self.get_dense_mask()

    def apply_mask_sparse(self, input_tensor):
        self._check_input(input_tensor)
        if self.is_full or self.is_empty:
            return input_tensor
        idx, _, data = self.get_index_mask()
        out = torch.zeros_like(input_tensor)
        if idx.numel() > 0:
            out.view(-1)[idx] = input_tensor.reshape(-1)[idx] * data
        return out

    def apply_inv_mask(self, input_tensor, mode: Literal["sparse", "dense"] = "dense"):
        if mode == "sparse":
            return self.apply_inv_mask_sparse(input_tensor)
        if mode == "dense":
            return self.apply_inv_mask_dense(input_tensor)
        raise ValueError(f"Invalid mode: {mode}")

    def apply_inv_mask_dense(self, input_tensor):
        self._check_input(input_tensor)
        if self.is_full or self.is_empty:
            return input_tensor
        dense = self.get_dense_mask()
        return input_tensor * (1.0 / (dense + 1e-6) * (dense != 0))

    def apply_inv_mask_sparse(self, input_tensor):
        self._check_input(input_tensor)
        if self.is_full or self.is_empty:
            return input_tensor
        idx, _, data = self.get_index_mask()
        out = torch.zeros_like(input_tensor)
        if idx.numel() > 0:
            out.view(-1)[idx] = input_tensor.reshape(-1)[idx] * (1.0 / (data + 1e-6))
        return out

    # ------------------------------------------------------------------ merge
    def merge_mask(self, other_mask: "Mask", inplace: bool,
                   mode: Literal["sparse", "dense"] = "dense") -> "Mask":
        if mode == "dense":
            return self.merge_mask_dense(other_mask, inplace)
        if mode == "sparse":
            return self.merge_mask_sparse(other_mask, inplace)
        raise ValueError(f"Invalid mode: {mode}")

    def _merge_trivial(self, other: "Mask", inplace: bool, index_form: bool) -> Optional["Mask"]:
        """Full / empty shortcuts shared by both merge modes; None when neither applies."""
        if self.shape != other.shape:
            raise ValueError(
                f"Cannot merge masks with different shapes: {self.shape} vs {other.shape}")
        if self.is_full or other.is_full:
            if not inplace:
                return Mask.create_full_mask(self.shape, self.dtype, self.device)
            self._reset_payload()
            self.is_full, self.is_empty = True, False
            self.from_dense_mask = self.from_index = False
            return self
        if self.is_empty and other.is_empty:
            return self if inplace else Mask.create_empty_mask(self.shape, self.dtype, self.device)
        if self.is_empty or other.is_empty:
            src = other if self.is_empty else self
            if inplace:
                if src is not self:
                    self._become(src)
                return self
            if index_form:
                idx, ptr, data = src.get_index_mask()
                return Mask.create_mask_from_indices(self.shape, idx, ptr, data, dtype=self.dtype)
            if src._native is not None and src._dense is None and src.dtype == self.dtype:
                return Mask._from_native(self.shape, self.dtype, src._native)  # bitmaps are not edited in place
            return Mask.create_mask_from_dense_mask(self.shape, src.get_dense_mask(),
                                                    dtype=self.dtype)
        return None

    def merge_mask_dense(self, other_mask: "Mask", inplace: bool) -> "Mask":
        done = self._merge_trivial(other_mask, inplace, index_form=False)
        if done is not None:
            return done
        if (self._native is not None and other_mask._native is not None and self._dense is None
                and other_mask._dense is None and self.dtype == other_mask.dtype):
            # both sides live as device bitmaps: merge there, no dense tensor
            from .._native_ops import merge_native

            merged_mask = merge_native(self, other_mask)
            if not inplace:
                return merged_mask
            self._become(merged_mask)
            return self
        merged = torch.clamp(self.get_dense_mask() + other_mask.get_dense_mask(), 0.0, 1.0)
        if not inplace:
            return Mask.create_mask_from_dense_mask(self.shape, merged, dtype=self.dtype)
        self._reset_payload()
        self._dense = merged
        self.from_dense_mask, self.from_index = True, False
        self.is_full = self.is_empty = False
        return self

    def merge_mask_sparse(self, other_mask: "Mask", inplace: bool) -> "Mask":
        done = self._merge_trivial(other_mask, inplace, index_form=True)
        if done is not None:
            return done
        rows, n = _n_rows(self.shape), self.shape[-1]
        a_idx, a_ptr, a_val = self.get_index_mask()
        b_idx, b_ptr, b_val = other_mask.get_index_mask()
        dev = a_idx.device if a_idx.numel() > 0 else b_idx.device
        if a_idx.numel() == 0 and b_idx.numel() == 0:
            idx = torch.empty(0, dtype=torch.long, device=dev)
            val = torch.empty(0, dtype=self.dtype, device=dev)
            ptr = torch.zeros(rows + 1, dtype=torch.long, device=dev)
        elif a_idx.numel() == 0 or b_idx.numel() == 0:
            idx, ptr, val = (b_idx, b_ptr, b_val) if a_idx.numel() == 0 else (a_idx, a_ptr, a_val)
            val = torch.clamp(val, 0.0, 1.0)
        elif a_idx.is_cuda and self.dtype in (torch.float32, torch.bfloat16):
            # the sums of equal indices in a float32 array over all positions, clamped and
            # rounded on the device; the ascending index form comes from the bitmap kernels
            lib = _native.load()
            st = _native.stream_of(dev)
            code = _native.dtype_code(self.dtype)
            total = rows * n
            acc = torch.zeros(total, dtype=torch.float32, device=dev)
            for i_, v_ in ((a_idx, a_val), (b_idx, b_val)):
                ic, vc = i_.to(torch.int64).contiguous(), v_.to(self.dtype).contiguous()
                _native.check(lib.sah_mask_flat_add(ic.data_ptr(), vc.data_ptr(), code, ic.numel(), total,
                                                    acc.data_ptr(), st), "sah_mask_flat_add")
            dense = torch.empty(tuple(self.shape), dtype=self.dtype, device=dev)
            _native.check(lib.sah_mask_clamp_to_dense(acc.data_ptr(), code, total, dense.data_ptr(), st),
                          "sah_mask_clamp_to_dense")
            idx, ptr, val = Mask.create_mask_from_dense_mask(self.shape, dense, self.dtype).get_index_mask()
        else:
            cat_idx = torch.cat([a_idx, b_idx])
            cat_val = torch.cat([a_val.to(self.dtype), b_val.to(self.dtype)])
            order = torch.argsort(cat_idx, stable=True)
            idx, inverse = torch.unique_consecutive(cat_idx[order], return_inverse=True)
            val = torch.zeros(idx.numel(), dtype=self.dtype, device=dev)
            val.scatter_add_(0, inverse, cat_val[order])
            val = torch.clamp(val, 0.0, 1.0)
            counts = torch.zeros(rows, dtype=torch.long, device=dev)
            counts.scatter_add_(0, idx // n, torch.ones_like(idx))
            ptr = torch.zeros(rows + 1, dtype=torch.long, device=dev)
            ptr[1:] = torch.cumsum(counts, dim=0)
        if not inplace:
            return Mask.create_mask_from_indices(self.shape, idx, ptr, val, dtype=self.dtype)
        self._reset_payload()
        self.indices, self.ptr, self.data = idx, ptr, val
        self.from_index, self.from_dense_mask = True, False
        self.is_full = self.is_empty = False
        return self

    # ---------------------------------------------------------------- density
    def get_density(self) -> float:
        if self.is_full:
            return 1.0
        if self.is_empty:
            return 0.0
        if self.from_dense_mask:
            if self._native is not None:
                nb = self._native
                nb.ensure_scan()
                return float(nb.ptr[-1].item()) / float(np.prod(self.shape))
            return float(torch.sum(self._dense > 0) / self._dense.numel())
        if self.from_index:
            return float(len(self.indices)) / float(np.prod(self.shape))
        raise RuntimeError("Mask object is in an invalid state")
