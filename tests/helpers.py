"""Shared helpers of the parity tests: synthetic inputs and un-tiling of operand records."""

from __future__ import annotations

import math

import numpy as np
import torch


def smooth_fields(frames, height, width, heads, dim, prefix, *, seed=0, outliers=(), dtype=torch.float16):
    """Seeded Q/K/V with the benchmark's statistics: Q and K are N(0,1) fields blurred per
    frame by a separable Gaussian (sigma = 2 tokens, reflect padding) plus 0.5 N(0,1); prefix
    rows and V are plain N(0,1); the channels in ``outliers`` of Q and K are scaled by 8."""
    gen = torch.Generator().manual_seed(seed)
    radius = 6
    taps = torch.exp(-0.5 * (torch.arange(-radius, radius + 1, dtype=torch.float32) / 2.0) ** 2)
    taps = taps / taps.sum()

    def field():
        x = torch.randn(frames, heads * dim, height, width, generator=gen)
        pad_h = min(radius, height - 1)
        pad_w = min(radius, width - 1)
        kh = taps[radius - pad_h : radius + pad_h + 1] / taps[radius - pad_h : radius + pad_h + 1].sum()
        kw = taps[radius - pad_w : radius + pad_w + 1] / taps[radius - pad_w : radius + pad_w + 1].sum()
        c = heads * dim
        x = torch.nn.functional.pad(x, (0, 0, pad_h, pad_h), mode="reflect") if pad_h else x
        x = torch.nn.functional.conv2d(x, kh.view(1, 1, -1, 1).expand(c, 1, -1, 1), groups=c)
        x = torch.nn.functional.pad(x, (pad_w, pad_w, 0, 0), mode="reflect") if pad_w else x
        x = torch.nn.functional.conv2d(x, kw.view(1, 1, 1, -1).expand(c, 1, 1, -1), groups=c)
        x = x + 0.5 * torch.randn(x.shape, generator=gen)
        x = x.permute(0, 2, 3, 1).reshape(frames * height * width, heads, dim)
        pre = torch.randn(prefix, heads, dim, generator=gen)
        x = torch.cat((pre, x), dim=0)
        for ch in outliers:
            x[..., ch] *= 8.0
        return x.unsqueeze(0)

    q = field()
    k = field()
    v = torch.randn(1, prefix + frames * height * width, heads, dim, generator=gen)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def untile(img: np.ndarray, rows: int, row_bytes: int) -> np.ndarray:
    """Core-matrix tile image (bytes) -> [rows, row_bytes] bytes."""
    chunks = row_bytes // 16
    return img.reshape(rows // 8, chunks, 8, 16).transpose(0, 2, 1, 3).reshape(rows, row_bytes)


def nibbles(packed: np.ndarray) -> np.ndarray:
    """[rows, n] packed bytes -> [rows, 2n] 4-bit codes, low nibble first."""
    out = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = packed & 0xF
    out[:, 1::2] = packed >> 4
    return out


def scale_block(blocks: np.ndarray, rows: int, ksteps: int) -> np.ndarray:
    """``ksteps`` 512-byte scale blocks -> [rows, 4*ksteps] scale bytes."""
    r = np.arange(rows)
    out = np.empty((rows, 4 * ksteps), dtype=np.uint8)
    for s in range(ksteps):
        for g in range(4):
            out[:, 4 * s + g] = blocks[s * 512 + (r % 32) * 16 + (r // 32) * 4 + g]
    return out


class Records:
    """Natural-order views of one head of an operand store (numpy, on the host)."""

    def __init__(self, store, shape, head: int):
        self.s = shape
        self.h = head
        self.b = {k: (None if v is None else v.detach().cpu().numpy()) for k, v in store.buffers.items()}
        self.D = shape.head_dim
        self.QB = shape.query_block
        self.R = shape.video_blocks
        self.NS = shape.stages

    def _rec(self, name, index, nbytes):
        return self.b[name].view(np.uint8)[index * nbytes : (index + 1) * nbytes]

    def q_fp16(self):
        n = self.QB * self.D * 2
        rows = [untile(self._rec("q_fp16", self.h * self.R + t, n), self.QB, self.D * 2).view(np.float16)
                for t in range(self.R)]
        return np.concatenate(rows)

    def kv_fp16(self):
        n = 2 * 64 * self.D * 2
        k, v = [], []
        for st in range(self.NS):
            r = self._rec("kv_fp16", self.h * self.NS + st, n)
            k.append(untile(r[: n // 2], 64, self.D * 2).view(np.float16))
            v.append(untile(r[n // 2 :], 64, self.D * 2).view(np.float16))
        return np.concatenate(k), np.concatenate(v)

    def q_int8(self, prefix=False):
        n = self.QB * self.D
        tiles = self.R + self.s.prefix_query_tiles
        rng = range(self.R, tiles) if prefix else range(self.R)
        rows = [untile(self._rec("q_int8", self.h * tiles + t, n), self.QB, self.D).view(np.int8) for t in rng]
        sc = self.b["q_int8_scale"].reshape(self.s.heads, tiles)[self.h]
        return np.concatenate(rows), (sc[self.R :] if prefix else sc[: self.R])

    def kv_int8(self):
        n = 2 * 64 * self.D
        k, v = [], []
        for st in range(self.NS):
            r = self._rec("kv_int8", self.h * self.NS + st, n)
            k.append(untile(r[: n // 2], 64, self.D).view(np.int8))
            v.append(untile(r[n // 2 :], self.D, 64).T)
        return (np.concatenate(k), self.b["k_int8_scale"].reshape(self.s.heads, self.NS)[self.h],
                np.concatenate(v), self.b["v_e4m3_scale"].reshape(self.s.heads, self.D)[self.h])

    def q_nvfp4(self):
        ks = self.D // 64
        n = self.QB * self.D // 2 + ks * 512
        codes, sf = [], []
        for t in range(self.R):
            r = self._rec("q_nvfp4", self.h * self.R + t, n)
            codes.append(nibbles(untile(r[: self.QB * self.D // 2], self.QB, self.D // 2)))
            sf.append(scale_block(r[self.QB * self.D // 2 :], self.QB, ks))
        return np.concatenate(codes), np.concatenate(sf)

    def kv_nvfp4(self):
        D = self.D
        ks = D // 64
        n = 64 * D + ks * 512 + 512
        kc, ksf, vc, vsf = [], [], [], []
        for st in range(self.NS):
            r = self._rec("kv_nvfp4", self.h * self.NS + st, n)
            kc.append(nibbles(untile(r[: 32 * D], 64, D // 2)))
            vc.append(nibbles(untile(r[32 * D : 64 * D], D, 32)).T)
            ksf.append(scale_block(r[64 * D : 64 * D + ks * 512], 64, ks))
            vsf.append(scale_block(r[64 * D + ks * 512 :], D, 1).T)          # [4, D]
        return np.concatenate(kc), np.concatenate(ksf), np.concatenate(vc), np.concatenate(vsf)


def compare_metrics(a: np.ndarray, b: np.ndarray):
    a = a.astype(np.float64).reshape(-1)
    b = b.astype(np.float64).reshape(-1)
    max_abs = float(np.abs(a - b).max())
    cos = float((a * b).sum() / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))
    rel = float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))
    return max_abs, cos, rel
