"""Line plots written as PNG files without a plotting library.

The reference's benchmarks save a PNG next to every CSV with matplotlib in its headless
mode (``benchmarks/collective_compare.py:7,74``, ``quantize_perf_curve.py``,
``stochastic_rounding_e2e_curve.py``, ``error_feedback_comparison.py``).  matplotlib is
used here too when it can be imported; otherwise a small rasteriser draws the same kind
of figure (axes, tick labels, one polyline per series, a legend) into an RGB buffer and
encodes it with ``zlib``: the benches keep their PNG output on machines that have
nothing but the standard library.
"""

from __future__ import annotations

import math
import struct
import zlib
from typing import Dict, List, Optional, Sequence, Tuple

Series = Dict[str, Tuple[Sequence[float], Sequence[float]]]  # label -> (xs, ys)

_COLORS = [(31, 119, 180), (255, 127, 14), (44, 160, 44), (214, 39, 40), (148, 103, 189),
           (140, 86, 75), (227, 119, 194), (127, 127, 127)]

# 5 x 7 bitmap font: rows top to bottom, 5 bits each
_FONT = {
    "0": "01110 10001 10011 10101 11001 10001 01110", "1": "00100 01100 00100 00100 00100 00100 01110",
    "2": "01110 10001 00001 00010 00100 01000 11111", "3": "11110 00001 00001 01110 00001 00001 11110",
    "4": "00010 00110 01010 10010 11111 00010 00010", "5": "11111 10000 11110 00001 00001 10001 01110",
    "6": "00110 01000 10000 11110 10001 10001 01110", "7": "11111 00001 00010 00100 01000 01000 01000",
    "8": "01110 10001 10001 01110 10001 10001 01110", "9": "01110 10001 10001 01111 00001 00010 01100",
    ".": "00000 00000 00000 00000 00000 01100 01100", "-": "00000 00000 00000 11111 00000 00000 00000",
    "+": "00000 00100 00100 11111 00100 00100 00000", "e": "00000 00000 01110 10001 11111 10000 01110",
    " ": "00000 00000 00000 00000 00000 00000 00000", "_": "00000 00000 00000 00000 00000 00000 11111",
    "/": "00001 00010 00010 00100 01000 01000 10000", "(": "00010 00100 01000 01000 01000 00100 00010",
    ")": "01000 00100 00010 00010 00010 00100 01000", ":": "00000 01100 01100 00000 01100 01100 00000",
    "%": "11001 11010 00010 00100 01000 01011 10011", ",": "00000 00000 00000 00000 00110 00100 01000",
    "=": "00000 00000 11111 00000 11111 00000 00000",
}
_LETTERS = {
    "a": "00000 00000 01110 00001 01111 10001 01111", "b": "10000 10000 10110 11001 10001 10001 11110",
    "c": "00000 00000 01110 10000 10000 10001 01110", "d": "00001 00001 01101 10011 10001 10001 01111",
    "f": "00110 01001 01000 11100 01000 01000 01000", "g": "00000 01111 10001 10001 01111 00001 01110",
    "h": "10000 10000 10110 11001 10001 10001 10001", "i": "00100 00000 01100 00100 00100 00100 01110",
    "j": "00010 00000 00110 00010 00010 10010 01100", "k": "10000 10000 10010 10100 11000 10100 10010",
    "l": "01100 00100 00100 00100 00100 00100 01110", "m": "00000 00000 11010 10101 10101 10001 10001",
    "n": "00000 00000 10110 11001 10001 10001 10001", "o": "00000 00000 01110 10001 10001 10001 01110",
    "p": "00000 00000 11110 10001 11110 10000 10000", "q": "00000 00000 01101 10011 01111 00001 00001",
    "r": "00000 00000 10110 11001 10000 10000 10000", "s": "00000 00000 01110 10000 01110 00001 11110",
    "t": "01000 01000 11100 01000 01000 01001 00110", "u": "00000 00000 10001 10001 10001 10011 01101",
    "v": "00000 00000 10001 10001 10001 01010 00100", "w": "00000 00000 10001 10001 10101 10101 01010",
    "x": "00000 00000 10001 01010 00100 01010 10001", "y": "00000 00000 10001 10001 01111 00001 01110",
    "z": "00000 00000 11111 00010 00100 01000 11111",
}
_FONT.update(_LETTERS)


class Canvas:
    def __init__(self, width: int, height: int):
        self.w, self.h = width, height
        self.px = bytearray([255]) * (3 * width * height)

    def dot(self, x: int, y: int, color):
        if 0 <= x < self.w and 0 <= y < self.h:
            i = 3 * (y * self.w + x)
            self.px[i:i + 3] = bytes(color)

    def line(self, x0, y0, x1, y1, color, thick: int = 1):
        x0, y0, x1, y1 = int(round(x0)), int(round(y0)), int(round(x1)), int(round(y1))
        dx, dy = abs(x1 - x0), -abs(y1 - y0)
        sx, sy = (1 if x0 < x1 else -1), (1 if y0 < y1 else -1)
        err = dx + dy
        while True:
            for t in range(thick):
                self.dot(x0, y0 + t, color)
                self.dot(x0 + t, y0, color)
            if x0 == x1 and y0 == y1:
                break
            e2 = 2 * err
            if e2 >= dy:
                err += dy
                x0 += sx
            if e2 <= dx:
                err += dx
                y0 += sy

    def text(self, x: int, y: int, s: str, color=(0, 0, 0), scale: int = 1):
        for ch in s:
            glyph = _FONT.get(ch) or _FONT.get(ch.lower()) or _FONT[" "]
            for r, row in enumerate(glyph.split()):
                for c, bit in enumerate(row):
                    if bit == "1":
                        for a in range(scale):
                            for b in range(scale):
                                self.dot(x + c * scale + a, y + r * scale + b, color)
            x += 6 * scale

    def png(self) -> bytes:
        raw = bytearray()
        stride = 3 * self.w
        for y in range(self.h):
            raw.append(0)
            raw += self.px[y * stride:(y + 1) * stride]

        def chunk(tag: bytes, data: bytes) -> bytes:
            body = tag + data
            return struct.pack(">I", len(data)) + body + struct.pack(">I", zlib.crc32(body))

        head = struct.pack(">IIBBBBB", self.w, self.h, 8, 2, 0, 0, 0)
        return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", head)
                + chunk(b"IDAT", zlib.compress(bytes(raw), 6)) + chunk(b"IEND", b""))


def _ticks(lo: float, hi: float, n: int = 5) -> List[float]:
    if hi <= lo:
        hi = lo + 1.0
    step = 10 ** math.floor(math.log10((hi - lo) / n))
    for m in (1, 2, 5, 10):
        if (hi - lo) / (step * m) <= n:
            step *= m
            break
    first = math.ceil(lo / step) * step
    out, v = [], first
    while v <= hi + 1e-12 * abs(hi):
        out.append(0.0 if abs(v) < step * 1e-9 else v)
        v += step
    return out


def _fmt(v: float) -> str:
    if v == 0:
        return "0"
    if abs(v) >= 1e5 or abs(v) < 1e-3:
        return f"{v:.1e}".replace("e+0", "e").replace("e-0", "e-").replace("e+", "e")
    return f"{v:.4g}"


def _rasterise(path: str, series: Series, title: str, xlabel: str, ylabel: str, logx: bool,
               logy: bool, size: Tuple[int, int]) -> None:
    W, H = size
    cv = Canvas(W, H)
    left, right, top, bottom = 70, 20, 30, 45

    def tx(v):
        return math.log10(v) if logx else v

    def ty(v):
        return math.log10(v) if logy else v

    pts = {k: [(tx(x), ty(y)) for x, y in zip(xs, ys)
               if math.isfinite(x) and math.isfinite(y) and (not logx or x > 0)
               and (not logy or y > 0)] for k, (xs, ys) in series.items()}
    allx = [p[0] for v in pts.values() for p in v] or [0.0, 1.0]
    ally = [p[1] for v in pts.values() for p in v] or [0.0, 1.0]
    x0, x1, y0, y1 = min(allx), max(allx), min(ally), max(ally)
    if x1 == x0:
        x1 = x0 + 1
    if y1 == y0:
        y1 = y0 + 1
    pad = 0.05 * (y1 - y0)
    y0, y1 = y0 - pad, y1 + pad

    def sx(v):
        return left + (v - x0) / (x1 - x0) * (W - left - right)

    def sy(v):
        return H - bottom - (v - y0) / (y1 - y0) * (H - top - bottom)

    grid, axis = (225, 225, 225), (60, 60, 60)
    for v in _ticks(x0, x1):
        cv.line(sx(v), top, sx(v), H - bottom, grid)
        label = _fmt(10 ** v if logx else v)
        cv.text(int(sx(v)) - 3 * len(label), H - bottom + 6, label)
    for v in _ticks(y0, y1):
        cv.line(left, sy(v), W - right, sy(v), grid)
        label = _fmt(10 ** v if logy else v)
        cv.text(max(2, left - 6 * len(label) - 4), int(sy(v)) - 3, label)
    cv.line(left, top, left, H - bottom, axis)
    cv.line(left, H - bottom, W - right, H - bottom, axis)
    for i, (name, p) in enumerate(pts.items()):
        color = _COLORS[i % len(_COLORS)]
        for a, b in zip(p, p[1:]):
            cv.line(sx(a[0]), sy(a[1]), sx(b[0]), sy(b[1]), color, thick=2)
        if len(p) <= 64:
            for a in p:
                for dx in (-2, -1, 0, 1, 2):
                    for dy in (-2, -1, 0, 1, 2):
                        cv.dot(int(sx(a[0])) + dx, int(sy(a[1])) + dy, color)
        ly = top + 4 + 11 * i
        cv.line(W - right - 150, ly + 3, W - right - 135, ly + 3, color, thick=2)
        cv.text(W - right - 130, ly, name[:21])
    cv.text(left, 8, title[:90], scale=1)
    cv.text(left + (W - left - right) // 2 - 3 * len(xlabel), H - 16, xlabel)
    cv.text(4, 8 + 11, ylabel[:10])
    with open(path, "wb") as f:
        f.write(cv.png())


def save_line_plot(path: str, series: Series, *, title: str = "", xlabel: str = "",
                   ylabel: str = "", logx: bool = False, logy: bool = False,
                   size: Tuple[int, int] = (900, 520), backend: Optional[str] = None) -> str:
    """Write ``series`` as a PNG line plot to ``path``; returns the backend that drew it
    ("matplotlib" or "builtin").  ``backend="builtin"`` forces the rasteriser."""
    if backend != "builtin":
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt

            fig, ax = plt.subplots(figsize=(size[0] / 100, size[1] / 100), dpi=100)
            for name, (xs, ys) in series.items():
                ax.plot(list(xs), list(ys), marker="o" if len(xs) <= 64 else None, label=name)
            if logx:
                ax.set_xscale("log")
            if logy:
                ax.set_yscale("log")
            ax.set_title(title)
            ax.set_xlabel(xlabel)
            ax.set_ylabel(ylabel)
            ax.grid(True, alpha=0.3)
            ax.legend()
            fig.tight_layout()
            fig.savefig(path)
            plt.close(fig)
            return "matplotlib"
        except ImportError:
            pass
    _rasterise(path, series, title, xlabel, ylabel, logx, logy, size)
    return "builtin"
