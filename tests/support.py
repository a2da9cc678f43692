"""Test helpers: typed access to the CPU oracle and the compiled reference."""

from __future__ import annotations

import ctypes as C
import hashlib
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
TILE_DTYPE = np.dtype([("expert_id", "<u4"), ("tile_m", "<u4"), ("tile_n", "<u4"),
                       ("valid_m", "<u4"), ("valid_n", "<u4")])

u32, u64, f64, vp = C.c_uint32, C.c_uint64, C.c_double, C.c_void_p


def sha(arr) -> str:
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()


def ptr(arr: np.ndarray):
    return arr.ctypes.data_as(vp)


def as_counts(counts) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(counts, dtype=np.uint32))


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = u + 0x7FFF + ((u >> 16) & 1)
    return (r >> 16).astype(np.uint16)


class Oracle:
    """oracle/liboracle.so (CPU restatement of the reference algorithms)."""

    def __init__(self) -> None:
        import build_oracle

        self.lib = C.CDLL(str(build_oracle.build_oracle()))
        self.lib.orc_build_tiles.restype = u64
        self.lib.orc_simulate.restype = u64
        self.lib.orc_probe_checksum.restype = u64
        self.lib.orc_grouped_gemm.restype = u64
        self.lib.orc_select_variant.restype = u32

    def generate_counts(self, experts, total_tokens, distribution, seed=2026, zipf_alpha=1.2,
                        heavy_fraction=0.1, heavy_share=0.8, inactive_fraction=0.5):
        out = np.zeros(max(1, experts), dtype=np.uint32)
        rc = self.lib.orc_generate_counts(u32(experts), u64(total_tokens), u32(distribution),
                                          u64(seed), f64(zipf_alpha), f64(heavy_fraction),
                                          f64(heavy_share), f64(inactive_fraction), ptr(out))
        return rc, out[:experts]

    def workload_metrics(self, counts, n, tile_m, tile_n):
        c = as_counts(counts)
        reals = np.zeros(6)
        ints = np.zeros(2, dtype=np.uint64)
        rc = self.lib.orc_workload_metrics(ptr(c), u32(len(c)), u32(n), u32(tile_m),
                                           u32(tile_n), ptr(reals), ptr(ints))
        return rc, reals, ints

    def build_tiles(self, counts, n, tile_m, tile_n, order=0, raster=0):
        c = as_counts(counts)
        total = self.lib.orc_build_tiles(ptr(c), u32(len(c)), u32(n), u32(tile_m), u32(tile_n),
                                         u32(order), u32(raster), None, u64(0))
        buf = np.zeros(max(1, total), dtype=TILE_DTYPE)
        self.lib.orc_build_tiles(ptr(c), u32(len(c)), u32(n), u32(tile_m), u32(tile_n),
                                 u32(order), u32(raster), ptr(buf), u64(total))
        return buf[:total]

    def simulate(self, scheduler, counts, n, tile_m, tile_n, cta_count):
        c = as_counts(counts)
        total = len(self.build_tiles(counts, n, tile_m, tile_n))
        tiles = np.zeros(max(1, total), dtype=TILE_DTYPE)
        offs = np.zeros(cta_count + 1, dtype=np.uint64)
        got = self.lib.orc_simulate(u32(scheduler), ptr(c), u32(len(c)), u32(n), u32(tile_m),
                                    u32(tile_n), u32(cta_count), ptr(tiles), ptr(offs))
        assert got == total
        ints = np.zeros(6, dtype=np.uint64)
        reals = np.zeros(6)
        self.lib.orc_schedule_metrics(ptr(tiles), ptr(offs), u32(cta_count), u32(tile_m),
                                      u32(tile_n), ptr(ints), ptr(reals))
        return tiles[:total], offs, ints, reals

    def routing_features(self, counts, n, tile_m, tile_n, cta_count):
        c = as_counts(counts)
        out = np.zeros(9)
        tiles = u64(0)
        rc = self.lib.orc_routing_features(ptr(c), u32(len(c)), u32(n), u32(tile_m),
                                           u32(tile_n), u32(cta_count), ptr(out), C.byref(tiles))
        return rc, out, int(tiles.value)

    def select_variant(self, tiles_per_cta, cv_m, inactive_ratio) -> int:
        return int(self.lib.orc_select_variant(f64(tiles_per_cta), f64(cv_m), f64(inactive_ratio)))

    def probe_checksum(self, tile_record, work_scale) -> int:
        rec = np.zeros(1, dtype=TILE_DTYPE)
        rec[0] = tuple(int(x) for x in tile_record)
        return int(self.lib.orc_probe_checksum(ptr(rec), u32(work_scale)))

    def combine_topk(self, src_bits, rows, weights=None):
        """src_bits [R, n] uint16, rows [T, top_k] int64, weights [T, top_k] f32 -> [T, n] uint16."""
        src_bits = np.ascontiguousarray(src_bits, dtype=np.uint16)
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        tokens, top_k = rows.shape
        n = src_bits.shape[1]
        if weights is not None:
            weights = np.ascontiguousarray(weights, dtype=np.float32)
            assert weights.shape == rows.shape
        out = np.zeros((tokens, n), dtype=np.uint16)
        rc = self.lib.orc_combine_topk(ptr(src_bits), C.c_uint64(src_bits.shape[0]), ptr(rows),
                                       ptr(weights) if weights is not None else None,
                                       C.c_uint64(tokens), u32(top_k), u32(n), ptr(out))
        assert rc == 0
        return out

    def e4m3_to_bf16(self, codes):
        """FP8 E4M3 bit patterns (uint8, any shape) -> the same values as BF16 bit patterns
        (exact: every E4M3 value is a BF16 value)."""
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        out = np.zeros(codes.shape, dtype=np.uint16)
        self.lib.orc_e4m3_to_bf16(ptr(codes), C.c_uint64(codes.size), ptr(out))
        return out

    def f32_to_e4m3(self, values):
        self.lib.orc_f32_to_e4m3.restype = C.c_uint8
        flat = np.ascontiguousarray(values, dtype=np.float32).ravel()
        return np.array([self.lib.orc_f32_to_e4m3(C.c_float(float(v))) for v in flat],
                        dtype=np.uint8).reshape(np.shape(values))

    def grouped_gemm(self, a_bits, w_bits, counts, n, k, *, want_f32=False, want_f64=False,
                     row_stride=1, row_phase=0, threads=0):
        """a_bits [sum M, k], w_bits [E, n, k] uint16 -> dict of outputs."""
        c = as_counts(counts)
        total = int(c.sum())
        a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
        w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
        assert a_bits.shape == (total, k) and w_bits.shape == (len(c), n, k)
        d = np.zeros((total, n), dtype=np.uint16)
        d32 = np.zeros((total, n), dtype=np.float32) if want_f32 else None
        d64 = np.zeros((total, n), dtype=np.float64) if want_f64 else None
        rows = self.lib.orc_grouped_gemm(
            ptr(a_bits), ptr(w_bits), ptr(c), u32(len(c)), u32(n), u32(k), ptr(d),
            ptr(d32) if want_f32 else None, ptr(d64) if want_f64 else None,
            u32(row_stride), u32(row_phase), C.c_int(threads))
        return {"bf16": d, "f32": d32, "f64": d64, "rows": int(rows)}


class RefLib:
    """oracle/_ref/libref_sched.so: the reference's own compiled host sources."""

    def __init__(self, path: Path) -> None:
        self.lib = C.CDLL(str(path))
        self.lib.ref_build_tiles.restype = u64
        self.lib.ref_simulate.restype = u64

    @classmethod
    def try_load(cls):
        import build_oracle

        path = build_oracle.build_reference()
        return cls(path) if path is not None and Path(path).exists() else None

    def generate_counts(self, experts, total_tokens, distribution, seed=2026, zipf_alpha=1.2,
                        heavy_fraction=0.1, heavy_share=0.8, inactive_fraction=0.5):
        out = np.zeros(max(1, experts), dtype=np.uint32)
        rc = self.lib.ref_generate_counts(u32(experts), u64(total_tokens), u32(distribution),
                                          u64(seed), f64(zipf_alpha), f64(heavy_fraction),
                                          f64(heavy_share), f64(inactive_fraction), ptr(out))
        return rc, out[:experts]

    def workload_metrics(self, counts, n, tile_m, tile_n):
        c = as_counts(counts)
        reals = np.zeros(6)
        ints = np.zeros(2, dtype=np.uint64)
        rc = self.lib.ref_workload_metrics(ptr(c), u32(len(c)), u32(n), u32(tile_m),
                                           u32(tile_n), ptr(reals), ptr(ints))
        return rc, reals, ints

    def build_tiles(self, counts, n, tile_m, tile_n, order=0):
        c = as_counts(counts)
        total = self.lib.ref_build_tiles(ptr(c), u32(len(c)), u32(n), u32(tile_m), u32(tile_n),
                                         u32(order), None, u64(0))
        if total == 2**64 - 1:
            return None
        buf = np.zeros(max(1, total), dtype=TILE_DTYPE)
        self.lib.ref_build_tiles(ptr(c), u32(len(c)), u32(n), u32(tile_m), u32(tile_n),
                                 u32(order), ptr(buf), u64(total))
        return buf[:total]

    def simulate(self, scheduler, counts, n, tile_m, tile_n, cta_count):
        c = as_counts(counts)
        total = len(self.build_tiles(counts, n, tile_m, tile_n))
        tiles = np.zeros(max(1, total), dtype=TILE_DTYPE)
        offs = np.zeros(cta_count + 1, dtype=np.uint64)
        ints = np.zeros(6, dtype=np.uint64)
        reals = np.zeros(6)
        got = self.lib.ref_simulate(u32(scheduler), ptr(c), u32(len(c)), u32(n), u32(tile_m),
                                    u32(tile_n), u32(cta_count), ptr(tiles), u64(total),
                                    ptr(offs), ptr(ints), ptr(reals))
        if got == 2**64 - 1:
            return None
        return tiles[:total], offs, ints, reals


# ------------------------------------------------------------ engine side --

def engine_host_tiles(engine, counts, n, tile_m, tile_n, order=0, raster=0) -> np.ndarray:
    tiles, total = engine.host_tiles(counts, n, tile_m, tile_n, order=order, raster=raster)
    return engine.tiles_to_numpy(tiles, total)


def engine_simulate(engine, scheduler, counts, n, tile_m, tile_n, cta_count):
    cap = engine._capi
    lib = cap.load()
    c = as_counts(counts)
    cp = c.ctypes.data_as(C.POINTER(C.c_uint32))
    total = lib.bmoe_host_tile_count(cp, len(c), n, tile_m, tile_n)
    if total == 2**64 - 1:  # zero tile dimension
        total = 0
    tiles = (cap.Tile * max(1, total))()
    offs = (C.c_uint64 * (cta_count + 1))()
    metrics = cap.ScheduleMetrics()
    rc = lib.bmoe_host_simulate(scheduler, cp, len(c), n, tile_m, tile_n, cta_count, tiles,
                                total, offs, C.byref(metrics))
    if rc != 0:
        return rc, None, None, None
    return rc, engine.tiles_to_numpy(tiles, total), np.asarray(list(offs), dtype=np.uint64), metrics


def kat_inputs(name: str):
    """Inputs of the reference's GEMM known-answer tests as BF16 bit patterns.

    Returns (counts, n, k, a_bits [sum M, k], w_bits [E, n, k]). Formulas:
    baselines/cutlass/test_correctness.cu:73-80,
    tests/test_sm100_dense_correctness.cu:62-69, tests/test_sm100_2sm_correctness.cu:61-68.
    """
    if name == "cutlass_baseline_kat":
        counts, n, k, div = [7, 0, 13, 31], 32, 32, 8.0
        fa = lambda i, e: (i + 3 * e) % 11 - 5
        fb = lambda i, e: (3 * i + e) % 13 - 6
    elif name == "sm100_dense_kat":
        counts, n, k, div = [128], 128, 64, 16.0
        fa = lambda i, e: i % 9 - 4
        fb = lambda i, e: (3 * i) % 11 - 5
    elif name == "sm100_2sm_kat":
        counts, n, k, div = [256], 128, 64, 16.0
        fa = lambda i, e: i % 7 - 3
        fb = lambda i, e: (5 * i) % 13 - 6
    else:
        raise KeyError(name)
    a_rows, w = [], np.zeros((len(counts), n, k), dtype=np.uint16)
    for e, m in enumerate(counts):
        ib = np.arange(n * k, dtype=np.int64)
        w[e] = f32_to_bf16_bits((fb(ib, e) / div).astype(np.float32)).reshape(n, k)
        if m:
            ia = np.arange(m * k, dtype=np.int64)
            a_rows.append(f32_to_bf16_bits((fa(ia, e) / div).astype(np.float32)).reshape(m, k))
    return counts, n, k, np.concatenate(a_rows, axis=0), w
