"""Checkpoint ingest: Hugging Face safetensors shards -> the packed expert buffer of a MoELayer.

The reference converts every shard to a .pt file, loads those into shared host memory and copies
expert by expert into per-expert GPU slots (moe_gen/models/deepseek/deepseek_parameter_server.py:176-223,
core/Parameter_Server/Parameter_Server.cpp:116-230), assigning tensors to parameters as they are
stored (moe_gen/models/deepseek/deepseekv3/deepseekv3_initializer.py:1005-1021).  Here the shards are
memory-mapped and one MoE layer's tensors go file -> pinned staging -> device staging -> packed buffer
(mg_pack_expert), two experts in flight, FP8 weights and their `weight_scale_inv` as stored.

The safetensors container: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the data.
"""
import json
import mmap
import os
import struct
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from . import lib as L

DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "F8_E4M3": (torch.float8_e4m3fn, 1),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}


class SafetensorsFile:
    """Read-only view of one shard; tensors are slices of the mapping, nothing is copied."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than 8 bytes)")
        (n,) = struct.unpack("<Q", head)
        size = os.fstat(self._f.fileno()).st_size
        if n <= 0 or 8 + n > size:
            raise ValueError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        meta = json.loads(self._f.read(n))
        self.metadata = meta.pop("__metadata__", {})
        self._base = 8 + n
        self.tensors: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in meta.items():
            dt, shape = info["dtype"], tuple(info["shape"])
            b, e = info["data_offsets"]
            if dt not in DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
            want = int(np.prod(shape, dtype=np.int64)) * DTYPES[dt][1]
            if e - b != want or b < 0 or self._base + e > size:
                raise ValueError(f"{path}: tensor {name} spans {e - b} bytes, shape {shape} {dt} needs {want}")
            self.tensors[name] = (dt, shape, b, e)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._bytes = np.frombuffer(self._map, dtype=np.uint8)

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a uint8 view of the mapping."""
        _, _, b, e = self.tensors[name]
        return self._bytes[self._base + b:self._base + e]

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.tensors[name]
        return DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU copy of the tensor (for small tensors and tests)."""
        dt, shape = self.info(name)
        raw = self.raw(name)
        if raw.size == 0:
            return torch.empty(shape, dtype=dt)
        return torch.from_numpy(raw.copy()).view(dt).view(shape)

    def close(self):
        self._bytes = None
        self._map.close()
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None):
    """Writes CPU tensors in the safetensors layout (data 8-byte aligned, names sorted)."""
    header, off, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} not supported")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


class Checkpoint:
    """Tensor name -> shard, over a directory or a list of .safetensors files.  Uses the
    `model.safetensors.index.json` weight map when the directory has one (so that only the shards a
    layer needs are opened), else reads every shard's header."""

    def __init__(self, source):
        if isinstance(source, (str, os.PathLike)) and os.path.isdir(source):
            self.dir = str(source)
            paths = sorted(os.path.join(self.dir, f) for f in os.listdir(self.dir) if f.endswith(".safetensors"))
        else:
            paths = [str(p) for p in ([source] if isinstance(source, (str, os.PathLike)) else source)]
            self.dir = os.path.dirname(paths[0]) if paths else "."
        if not paths:
            raise FileNotFoundError(f"no .safetensors files in {source}")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        index = os.path.join(self.dir, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                for name, shard in json.load(f)["weight_map"].items():
                    self._where[name] = os.path.join(self.dir, shard)
        else:
            for p in paths:
                for name in self._open(p).tensors:
                    self._where[name] = p

    def _open(self, path: str) -> SafetensorsFile:
        if path not in self._files:
            self._files[path] = SafetensorsFile(path)
        return self._files[path]

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def file_of(self, name: str) -> SafetensorsFile:
        if name not in self._where:
            raise KeyError(f"tensor {name} is not in the checkpoint")
        return self._open(self._where[name])

    def close(self):
        for f in self._files.values():
            f.close()
        self._files.clear()


# tensor names of one MoE block: (router weight, router bias or None, expert pattern, (gate, up, down), shared)
NAMING = {
    "deepseek": ("{p}.mlp.gate.weight", "{p}.mlp.gate.e_score_correction_bias", "{p}.mlp.experts.{e}.{m}",
                 ("gate_proj", "up_proj", "down_proj"), "{p}.mlp.shared_experts.{m}"),
    "mixtral": ("{p}.block_sparse_moe.gate.weight", None, "{p}.block_sparse_moe.experts.{e}.{m}",
                ("w1", "w3", "w2"), None),
}


def _copy_into(dst: np.ndarray, src: np.ndarray):
    np.copyto(dst, src)          # releases the GIL: several of these run on pool threads


def load_moe_layer(layer, checkpoint: Checkpoint, layer_idx: int, naming: str = "deepseek",
                   prefix: str = "model.layers.{}", n_threads: int = 8) -> dict:
    """Fills `layer` (a MoELayer, any ep_rank) with block `layer_idx` of the checkpoint: router, this
    rank's experts, shared expert.  Returns byte and time counts.  Expert matrices must be stored in
    the layer's weight format (FP8 e4m3 + `weight_scale_inv` for MG_WEIGHT_FP8_BLOCK128, else bf16); an
    FP8-stored shared expert is de-quantised on the device, since the packed layout keeps it bf16."""
    gate_n, bias_n, exp_n, mats, shared_n = NAMING[naming]
    p = prefix.format(layer_idx)
    dev = layer.device
    fp8 = layer.desc.weight_format == L.WEIGHT_FP8_BLOCK128
    t_start = time.perf_counter()
    nbytes = 0

    gw = checkpoint.file_of(gate_n.format(p=p)).tensor(gate_n.format(p=p))
    bias = None
    if bias_n is not None and bias_n.format(p=p) in checkpoint:
        bias = checkpoint.file_of(bias_n.format(p=p)).tensor(bias_n.format(p=p)).float()
    layer.set_router(gw.to(torch.bfloat16), bias)
    nbytes += gw.numel() * gw.element_size()

    # ---- routed experts: 3 matrices (+3 scale tensors) per expert through two staging sets
    def pieces(e: int) -> List[Tuple[SafetensorsFile, str]]:
        out = []
        for m in mats:
            n = exp_n.format(p=p, e=e, m=m) + ".weight"
            out.append((checkpoint.file_of(n), n))
        if fp8:
            for m in mats:
                n = exp_n.format(p=p, e=e, m=m) + ".weight_scale_inv"
                out.append((checkpoint.file_of(n), n))
        return out

    I, H = layer.I, layer.H
    wdt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    want = [((I, H), wdt), ((I, H), wdt), ((H, I), wdt)]
    if fp8:
        want += [((-(-I // 128), -(-H // 128)), torch.float32)] * 2 + [((-(-H // 128), -(-I // 128)), torch.float32)]
    sizes = [int(np.prod(s)) * torch.empty(0, dtype=d).element_size() for s, d in want]
    offs = np.concatenate([[0], np.cumsum([(s + 255) // 256 * 256 for s in sizes])]).astype(np.int64)
    total = int(offs[-1])
    with torch.cuda.device(dev):
        pinned = [torch.empty(total, dtype=torch.uint8).pin_memory() for _ in range(2)]
        staged = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(2)]
        copy_stream = torch.cuda.Stream(device=dev)
        copied = [torch.cuda.Event() for _ in range(2)]
        packed = [torch.cuda.Event() for _ in range(2)]
        comp = torch.cuda.current_stream(dev)
        pool = ThreadPoolExecutor(max_workers=max(1, n_threads))
        try:
            for i in range(layer.e_local):
                e, b = layer.expert_lo + i, i & 1
                src = pieces(e)
                for (f, n), (shape, dt) in zip(src, want):
                    got_dt, got_shape = f.info(n)
                    if got_dt != dt or tuple(got_shape) != tuple(shape):
                        raise ValueError(f"{n}: stored as {tuple(got_shape)} {got_dt}, the layer needs {tuple(shape)} {dt}")
                if i >= 2:
                    copied[b].synchronize()            # the pinned set is free once its copy has run
                host = pinned[b].numpy()
                futs = []
                for j, (f, n) in enumerate(src):
                    raw = f.raw(n)
                    # large matrices in slices so that the pool's threads share them
                    step = max(1 << 20, -(-raw.size // max(1, n_threads)))
                    for a in range(0, raw.size, step):
                        z = min(raw.size, a + step)
                        futs.append(pool.submit(_copy_into, host[offs[j] + a:offs[j] + z], raw[a:z]))
                for fu in futs:
                    fu.result()
                with torch.cuda.stream(copy_stream):
                    if i >= 2:
                        copy_stream.wait_event(packed[b])  # the device set is free once its expert is packed
                    staged[b].copy_(pinned[b], non_blocking=True)
                    copied[b].record(copy_stream)
                comp.wait_event(copied[b])
                base = staged[b].data_ptr()
                ptrs = [base + int(o) for o in offs[:-1]]
                sc = ptrs[3:6] if fp8 else [None, None, None]
                L.check(layer.lib.mg_pack_expert(layer._h, i, ptrs[0], ptrs[1], ptrs[2], sc[0], sc[1], sc[2],
                                                 layer.packed.data_ptr(), comp.cuda_stream))
                packed[b].record(comp)
                nbytes += sum(sizes)
            comp.synchronize()
        finally:
            pool.shutdown(wait=True)

    # ---- shared expert (bf16 in the packed layout)
    if layer.Is and shared_n is not None:
        ws = []
        for m in mats:
            n = shared_n.format(p=p, m=m) + ".weight"
            f = checkpoint.file_of(n)
            t = f.tensor(n)
            nbytes += t.numel() * t.element_size()
            if t.dtype == torch.float8_e4m3fn:
                sn = shared_n.format(p=p, m=m) + ".weight_scale_inv"
                s = checkpoint.file_of(sn).tensor(sn)
                t = layer.dequant_fp8(t.to(dev), s.to(dev))
            ws.append(t.to(torch.bfloat16))
        layer.load_shared(*ws)
    dt = time.perf_counter() - t_start
    return {"bytes": int(nbytes), "seconds": dt, "gb_per_s": nbytes / dt / 1e9, "experts": layer.e_local}


def export_moe_layer(path: str, layer_idx: int, gate_w: torch.Tensor, bias: Optional[torch.Tensor],
                     experts: Iterable[Tuple], shared: Optional[Tuple] = None, naming: str = "deepseek",
                     prefix: str = "model.layers.{}"):
    """Writes one MoE block in the checkpoint's naming (tests, and tools that build synthetic
    checkpoints).  experts: per expert (gate, up, down) bf16 matrices, or for FP8 checkpoints
    ((q, scale_inv), (q, scale_inv), (q, scale_inv))."""
    gate_n, bias_n, exp_n, mats, shared_n = NAMING[naming]
    p = prefix.format(layer_idx)
    out = {gate_n.format(p=p): gate_w}
    if bias is not None and bias_n is not None:
        out[bias_n.format(p=p)] = bias
    for e, ws in enumerate(experts):
        for m, w in zip(mats, ws):
            n = exp_n.format(p=p, e=e, m=m)
            if isinstance(w, (tuple, list)):
                out[n + ".weight"], out[n + ".weight_scale_inv"] = w[0], w[1]
            else:
                out[n + ".weight"] = w
    if shared is not None and shared_n is not None:
        for m, w in zip(mats, shared):
            out[shared_n.format(p=p, m=m) + ".weight"] = w
    write_safetensors(path, out)
