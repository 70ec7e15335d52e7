"""The B200 (sm_100a) device description the scheduler side needs, with the attribute names of the
reference's ``Arch`` / ``CUDA`` classes (python/cleave/arch/arch_base.py:4-41, python/cleave/arch/cuda.py:120-186),
plus what is new on this architecture: tensor memory and the tcgen05 instruction shapes.

The reference scores tilings against these fields (shared-memory capacity, SM count, L2 size, tensor
instruction shapes) and has rows for sm_90 only; ``OFFLINE_DEVICES`` below is the sm_100 row in the same
format, and ``snap_tile`` maps a plan's tile hint onto the tile shapes the hand-written kernels implement,
so that plans scheduled with this description arrive already snapped.
"""

from __future__ import annotations

from dataclasses import dataclass, field

# Same shape as python/cleave/arch/cuda.py:121-123 (limits used when no GPU is visible).
OFFLINE_DEVICES = {
    100: {"name": "offline sm_100 (B200 limits)", "sms": 148, "l2": 126 * 2**20},
}


@dataclass(frozen=True)
class TensorInstruction:
    """``name`` and the (M, N) extent of one instruction, as python/cleave/arch/cuda.py:111-118."""

    name: str
    shape: tuple


# tcgen05.mma kind::f16: M 128 per CTA (256 across a CTA pair), N a multiple of 16 up to 256, K 16.
TCGEN05_SHAPES = (
    TensorInstruction("tcgen05.cta_group::1", (128, 128)),
    TensorInstruction("tcgen05.cta_group::1", (128, 256)),
    TensorInstruction("tcgen05.cta_group::2", (256, 256)),
)

# Output tiles (rows, columns) of the GEMM kernels: single-CTA tiles and the CTA-pair tile.
KERNEL_TILES = ((128, 128), (128, 256), (256, 256))


@dataclass
class B200:
    """Field for field the reference's ``CUDA`` description, filled in for one B200."""

    name: str = "NVIDIA B200"
    platform: str = "CUDA"
    sm_version: int = 100
    compute_capability: str = "100"
    compute_max_core: int = 148            # SMs (two dies of 74)
    warp_size: int = 32
    sm_partition: int = 4
    reg_cap: int = 65536                   # 32-bit registers per SM
    smem_cap: int = 227 * 2**10            # opt-in dynamic shared memory per CTA
    max_smem_usage: int = 227 * 2**10      # one CTA per SM is the design point of these kernels
    l2_cache_size_bytes: int = 126 * 2**20
    transaction_size: list = field(default_factory=lambda: [32, 128])
    bandwidth: list = field(default_factory=lambda: [6537, 90000])  # GB/s: HBM (measured copy), L2 -> SM aggregate
    tmem_columns: int = 512                # 32-bit columns x 128 lanes of tensor memory per SM (256 KB)
    hbm_bytes: int = 180 * 10**9
    k_step: int = 16                       # K extent of one tcgen05.mma for 16-bit operands
    tensorcore_supported: tuple = (("float16", "float32"), ("bfloat16", "float32"))

    def get_avaliable_tensorintrin_shapes(self):  # the reference's spelling
        return [list(t.shape) for t in TCGEN05_SHAPES]

    def is_tensorcore_supported_precision(self, in_dtype: str, accum_dtype: str) -> bool:
        return (in_dtype, accum_dtype) in self.tensorcore_supported


def snap_tile(rows: int, cols: int, m: int | None = None, n: int | None = None) -> tuple:
    """The kernel tile closest to a plan's ``output_tile`` hint (rows x cols of one CTA's output). Hints come
    from a scheduler that scored them for another architecture (e.g. 64 x 32 for the split-K matmul partial);
    the kernels implement ``KERNEL_TILES`` only. The smallest kernel tile that covers the hint is taken,
    capped by the problem's own extent when ``m`` / ``n`` are given (a 64-row problem never needs the
    256-row pair tile)."""
    if rows <= 0 or cols <= 0:
        raise ValueError("tile extents must be positive")
    for tr, tc in KERNEL_TILES:
        if m is not None and tr > 128 and m < 512:
            continue  # the pair kernel takes M >= 512 only
        if tr >= rows and tc >= cols:
            return (tr, tc)
        if n is not None and tc >= n and tr >= rows:
            return (tr, tc)
    fits = [t for t in KERNEL_TILES if m is None or t[0] <= 128 or m >= 512]
    return fits[-1]


def tmem_columns_needed(tile: tuple, accumulators: int = 2) -> int:
    """Tensor-memory columns one CTA needs for ``accumulators`` fp32 accumulators of ``tile``: every CTA
    holds 128 rows (its half of a pair tile) by all of the tile's columns, one 32-bit column each. The
    GEMM kernels double-buffer the accumulator so that the epilogue of one tile overlaps the main loop of
    the next; 2 x 256 columns fills the 512 columns of an SM."""
    return accumulators * tile[1]


class TCPolicyB200:
    """Scores GEMM-family plans for sm_100 with the cost model the kernels themselves plan by (the role of the
    reference's ``TCPolicy``, python/cleave/schedule/policy/default.py:1015-1110, which scores tilings for sm_90).
    A candidate here is what the backend honours of a plan: operator, extents and split factor; the score is the
    model's estimate in microseconds for the tile, cluster or pair plan the library would run for it. It needs the
    built library and a visible GPU (the plan depends on the SM count and on how many clusters fit at once)."""

    KIND = {0: "tiles", 1: "cluster split-K", 2: "CTA pairs"}
    OPS = {"matmul": 0, "rmsnorm_matmul": 1, "swiglu": 2}

    def plan(self, family: str, dims: dict, dtype: str = "float16", split: int = 0) -> dict:
        import ctypes as C

        from . import _lib

        a, info = _lib.GemmArgs(), _lib.GemmPlanInfo()
        a.m, a.n, a.k, a.op = int(dims["M"]), int(dims["N"]), int(dims["K"]), self.OPS[family]
        a.dtype, a.split_k = (_lib.F16 if dtype in ("float16", "f16") else _lib.BF16), int(split if split > 1 else 0)
        _lib.check(_lib.lib().cb200_gemm_plan(C.byref(a), C.byref(info)))
        return {"tile": (info.tile_m, info.tile_n), "split": info.split, "kind": self.KIND[info.kind], "grid": info.grid,
                "estimate_us": float(info.estimate_us)}

    def rank(self, specs) -> list:
        """``[(estimate_us, spec)]`` for kernel specs of the GEMM family, best first: the order a scheduler should
        offer its candidates in, instead of the order an sm_90 policy scored them in."""
        scored = [(self.plan(s.family, s.dims, s.dtype, s.split)["estimate_us"], i, s) for i, s in enumerate(specs)
                  if s.family in self.OPS]
        return [(us, s) for us, _, s in sorted(scored)]
