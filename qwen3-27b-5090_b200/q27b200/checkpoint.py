"""NVFP4 projections from a safetensors checkpoint into the buffers the kernels read: the loading side of the engine's
weight records (Weights::fp4 / fp4_glu / fuse, engine/src/weights.cc:125-141,177-185,254-314) on top of the library's
q27b_ckpt_* entry points. Both on-disk namings are read (modelopt: weight, weight_scale, weight_scale_2, input_scale;
compressed-tensors: weight_packed, weight_scale, weight_global_scale = 1 / weight_scale_2, input_global_scale =
1 / input_scale). The file goes through pinned staging straight to the device; the block scales are swizzled and the
gate | up rows interleaved on the way (strided copies and one kernel), nothing is re-laid-out on the host.

`write_safetensors` produces such files (tests, and exporting synthetic weights)."""

from __future__ import annotations

import ctypes
import json
import struct

import numpy as np
import torch

from . import layouts
from .linear import Fp4Linear, Fp4Mlp
from .q27lib import call, last_error, lib


class Fp4LayerInfo(ctypes.Structure):
    """Mirror of q27b_fp4_layer (include/q27b200/capi.h)."""

    _fields_ = [("out", ctypes.c_int), ("inp", ctypes.c_int), ("w_scale2", ctypes.c_float), ("in_scale", ctypes.c_float),
                ("compressed_tensors", ctypes.c_int)]


class Checkpoint:
    """An open checkpoint (a .safetensors file or a directory of shards)."""

    def __init__(self, path: str):
        self._h = ctypes.c_void_p()
        call("q27b_ckpt_open", str(path).encode(), ctypes.byref(self._h))
        self._scratch: torch.Tensor | None = None

    def close(self):
        if self._h:
            lib().q27b_ckpt_close(self._h)
            self._h = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        self.close()

    def __len__(self) -> int:
        return lib().q27b_ckpt_count(self._h)

    def tensor_info(self, name: str):
        """(dtype string, shape tuple, bytes) or None if the checkpoint has no such tensor."""
        dtype = ctypes.create_string_buffer(16)
        shape = (ctypes.c_int64 * 8)()
        ndim, nbytes = ctypes.c_int(), ctypes.c_int64()
        rc = lib().q27b_ckpt_tensor(self._h, name.encode(), dtype, 16, shape, 8, ctypes.byref(ndim), ctypes.byref(nbytes))
        if rc == 1:
            return None
        if rc:
            raise RuntimeError(last_error())
        return dtype.value.decode(), tuple(shape[i] for i in range(ndim.value)), nbytes.value

    def has(self, name: str) -> bool:
        return self.tensor_info(name) is not None

    def read(self, name: str) -> np.ndarray:
        """The raw bytes of a tensor (host)."""
        info = self.tensor_info(name)
        if info is None:
            raise KeyError(name)
        buf = np.empty(info[2], dtype=np.uint8)
        call("q27b_ckpt_read", self._h, name.encode(), 0, info[2], buf)
        return buf

    def fp4_layer(self, prefix: str) -> Fp4LayerInfo:
        info = Fp4LayerInfo()
        call("q27b_ckpt_fp4_layer", self._h, prefix.encode(), ctypes.byref(info))
        return info

    def _scratch_for(self, nbytes: int, device) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < nbytes or self._scratch.device != torch.device(device):
            self._scratch = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        return self._scratch

    def _upload(self, prefix: str, half: int, w: torch.Tensor, sf: torch.Tensor, info: Fp4LayerInfo):
        scratch = self._scratch_for(info.out * info.inp // 16, w.device)
        call("q27b_ckpt_load_fp4", self._h, prefix.encode(), half, w, sf, scratch, scratch.numel(),
             torch.cuda.current_stream().cuda_stream)

    def load_fp4(self, prefix: str, device="cuda", workspace: torch.Tensor | None = None) -> Fp4Linear:
        """One projection (Weights::fp4)."""
        li = self.fp4_layer(prefix)
        assert li.out % 128 == 0 and li.inp % 64 == 0, f"{prefix}: [{li.out}][{li.inp}] is not a shape the GEMMs take"
        w = torch.empty(li.out, li.inp // 2, dtype=torch.uint8, device=device)
        sf = torch.zeros(layouts.sf_bytes(li.out, li.inp // 16), dtype=torch.uint8, device=device)
        self._upload(prefix, -1, w, sf, li)
        return Fp4Linear(w, sf, li.w_scale2, li.in_scale, li.out, li.inp, False, workspace)

    def load_fp4_fused(self, prefixes: list[str], device="cuda", workspace: torch.Tensor | None = None) -> Fp4Linear:
        """Projections that read the same activation, loaded back to back into one weight with one alpha per part
        (fuse4, engine/src/weights.cc:254-267: same reduction length, same input scale, every part a multiple of 128
        rows so that the scale atoms are adjacent too)."""
        infos = [self.fp4_layer(p) for p in prefixes]
        assert 2 <= len(infos) <= 4, "two to four parts"
        assert all(i.inp == infos[0].inp for i in infos), "fused NVFP4 layers differ in their input width"
        assert all(i.in_scale == infos[0].in_scale for i in infos), "fused NVFP4 layers have different input scales"
        assert all(i.out % 128 == 0 for i in infos), "every fused part must be a multiple of 128 rows"
        K, rows = infos[0].inp, sum(i.out for i in infos)
        w = torch.empty(rows, K // 2, dtype=torch.uint8, device=device)
        sf = torch.zeros(layouts.sf_bytes(rows, K // 16), dtype=torch.uint8, device=device)
        r = 0
        for p, li in zip(prefixes, infos):
            self._upload(p, -1, w[r:], sf[layouts.sf_bytes(r, K // 16):], li)
            r += li.out
        f = Fp4Linear(w, sf, infos[0].w_scale2, infos[0].in_scale, rows, K, False, workspace)
        f._w_scales = [i.w_scale2 for i in infos]
        begins = [sum(i.out for i in infos[:j]) for j in range(len(infos))]
        f._set_segments(begins, [f.in_scale * g for g in f._w_scales])
        return f

    def load_fp4_glu(self, gate: str, up: str, device="cuda", workspace: torch.Tensor | None = None):
        """The gate and the up projection of an MLP as ONE interleaved gate | up weight (Weights::fp4_glu). Returns
        (Fp4Linear with glu=True, alpha_gate, alpha_up): the two keep their own tensor scales, which the SiLU*mul
        epilogue applies (engine/src/weights.cc:302-310, model.cc:1062-1064)."""
        g, u = self.fp4_layer(gate), self.fp4_layer(up)
        assert g.out == u.out and g.inp == u.inp and g.out % 128 == 0 and g.inp % 64 == 0, "unexpected MLP gate / up"
        assert g.in_scale == u.in_scale, "MLP gate / up have different input scales"
        w = torch.empty(2 * g.out, g.inp // 2, dtype=torch.uint8, device=device)
        sf = torch.zeros(layouts.sf_bytes(2 * g.out, g.inp // 16), dtype=torch.uint8, device=device)
        self._upload(gate, 0, w, sf, g)
        self._upload(up, 1, w, sf, u)
        lin = Fp4Linear(w, sf, g.w_scale2, g.in_scale, g.out, g.inp, True, workspace)
        lin.w_scale2_gate, lin.w_scale2_up = float(g.w_scale2), float(u.w_scale2)
        lin.set_in_scale(g.in_scale)
        return lin, lin.alpha_gate, lin.alpha_up

    def load_mlp(self, prefix: str, device="cuda", workspace: torch.Tensor | None = None) -> Fp4Mlp:
        """<prefix>.gate_proj / .up_proj / .down_proj as the engine's MLP."""
        gu, ag, au = self.load_fp4_glu(f"{prefix}.gate_proj", f"{prefix}.up_proj", device, workspace)
        down = self.load_fp4(f"{prefix}.down_proj", device, gu.ws)
        return Fp4Mlp(gu, down, ag, au)


_DTYPES = {"U8": np.uint8, "F32": np.float32, "I32": np.int32, "I64": np.int64, "F8_E4M3": np.uint8, "BF16": np.uint16}


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None):
    """tensors: name -> (dtype string, numpy array whose bytes are stored as they are; F8_E4M3 as uint8 codes, BF16 as
    uint16 bit patterns). Tensor data is 8-byte aligned as the format asks."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, (dtype, arr) in tensors.items():
        arr = np.ascontiguousarray(arr)
        assert arr.dtype == _DTYPES[dtype], f"{name}: {arr.dtype} for {dtype}"
        raw = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def fp4_tensors(prefix: str, codes: np.ndarray, sf_rowmajor: np.ndarray, w_scale2: float, in_scale: float,
                compressed_tensors: bool = False) -> dict:
    """The four tensors of one projection in the chosen naming (for write_safetensors)."""
    one = lambda v: np.array([v], dtype=np.float32)  # noqa: E731
    if compressed_tensors:
        return {f"{prefix}.weight_packed": ("U8", codes), f"{prefix}.weight_scale": ("F8_E4M3", sf_rowmajor),
                f"{prefix}.weight_global_scale": ("F32", one(np.float32(1.0) / np.float32(w_scale2))),
                f"{prefix}.input_global_scale": ("F32", one(np.float32(1.0) / np.float32(in_scale)))}
    return {f"{prefix}.weight": ("U8", codes), f"{prefix}.weight_scale": ("F8_E4M3", sf_rowmajor),
            f"{prefix}.weight_scale_2": ("F32", one(w_scale2)), f"{prefix}.input_scale": ("F32", one(in_scale))}
