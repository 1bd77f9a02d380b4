"""Static geometry of a Buffer: slot capacity, limits and heap layout.

The capacity rule follows the reference (moonep/api.py:265-279): a destination
rank holds at most ``epn`` local plus ``epn`` remote non-empty expert segments,
each padded to ``token_padding`` rows, so
``NvS = align_up(S*K + (token_padding-1)*2*epn, token_padding)``.
Limits mirror planning.py:1231-1255 / dispatch.py:761-784 of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

INT32_MAX = 2**31 - 1
MAX_RANKS = 128          # 7 rank bits in the reference's encodings (constants.py:7)
MAX_TOPK = 32            # per-token duplicate bitmask width
MAX_NVS = (1 << 24) - 1  # slot offsets fit 24 bits
MAX_VRANKS = 8           # ranks one process may host in single-GPU emulation
VBLOCK = 1024            # planning kernel block size (entries ranked per CTA pass)
FLAG_ROWS = 128          # rows per ready-flag tile (the grouped GEMM's M tile)


def align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass(frozen=True)
class Geometry:
    S: int
    H: int
    K: int
    E: int
    R: int
    token_padding: int
    num_sms: int

    # derived
    epn: int = 0
    N: int = 0
    NvS: int = 0
    vblock_entries: int = 0   # entries per planning vblock (multiple of K)
    num_vblocks: int = 0

    # byte offsets inside one rank's symmetric heap chunk
    off_hidden: int = 0
    off_weights: int = 0
    off_tpe: int = 0
    off_bar: int = 0
    off_dupcnt: int = 0
    off_dupgroups: int = 0
    off_duploffs: int = 0
    off_ready: int = 0        # uint32 [ntiles] arrival counters of the ready-flag tiles
    off_rowsrc: int = 0       # int32 [NvS] slot a row's payload comes from (flagged dispatch)
    ntiles: int = 0           # ceil(NvS / FLAG_ROWS)
    off_slotflag: int = 0     # uint32 [epn] prefetch epoch at which each prefetch slot of this rank became complete
    off_srcinfo: int = 0      # push-combine only (0 = not allocated): provenance table [NvS] int32,
    off_push: int = 0         # receive area [S*K, H] bf16,
    off_pushw: int = 0        # per-slot scalar receive area [S*K] fp32
    dup_group_cap: int = 0    # staging capacity per source rank (groups)
    dup_loff_cap: int = 0     # staging capacity per source rank (duplicate offsets)
    chunk_bytes: int = 0      # before granularity padding

    @staticmethod
    def make(S, H, K, E, R, token_padding=128, num_sms=32, push_combine=False) -> "Geometry":
        for name, v in (("S", S), ("H", H), ("K", K), ("E", E), ("num_ep_ranks", R)):
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ValueError(f"{name} must be a positive int, got {v!r}")
        assert isinstance(token_padding, int) and token_padding > 0, \
            f"token_padding must be a positive int, got {token_padding}"
        assert E % R == 0, f"E ({E}) must be divisible by R ({R})"
        epn = E // R
        N = S * K
        assert 0 < N < INT32_MAX, f"planning requires 0 < S*K < int32_max, got {N}"
        NvS = align_up(N + (token_padding - 1) * 2 * epn, token_padding)
        assert R <= MAX_RANKS, f"R <= {MAX_RANKS} required, got {R}"
        assert K <= MAX_TOPK, f"K <= {MAX_TOPK} required, got {K}"
        assert NvS <= MAX_NVS, f"NvS <= {MAX_NVS} required, got {NvS}"
        assert R * NvS <= INT32_MAX, f"R*NvS must fit int32, got {R * NvS}"
        assert H % 8 == 0, f"H must be a multiple of 8 (16-byte rows), got {H}"
        vb = (VBLOCK // K) * K
        nvb = (N + vb - 1) // vb

        off = 0

        def take(nbytes, align=1024):
            nonlocal off
            off = align_up(off, align)
            start = off
            off += nbytes
            return start

        o_hidden = take(NvS * H * 2)
        o_weights = take(NvS * 4)
        o_tpe = take(R * E * 4)
        o_bar = take(4 * MAX_RANKS * 4)       # 4 independent flag rows
        # duplicate-group staging: one region per SOURCE rank, so senders never contend.
        # A source can emit at most N/2 groups and N duplicate offsets to one destination.
        gcap, lcap = N // 2 + 1, N
        o_dupcnt = take(R * 2 * 4)
        o_dupgroups = take(R * gcap * 3 * 4)
        o_duploffs = take(R * lcap * 4)
        ntiles = (NvS + FLAG_ROWS - 1) // FLAG_ROWS
        o_ready = take(4 * ntiles)
        o_rowsrc = take(4 * NvS)
        o_slotflag = take(4 * epn)
        o_srcinfo = o_push = o_pushw = 0
        if push_combine:
            # the expert GEMM's epilogue sends every output row back to its source rank
            o_srcinfo = take(NvS * 4)
            o_push = take(N * H * 2)
            o_pushw = take(N * 4)
        chunk = align_up(off, 1024)
        return Geometry(S, H, K, E, R, token_padding, num_sms, epn, N, NvS, vb, nvb,
                        o_hidden, o_weights, o_tpe, o_bar, o_dupcnt, o_dupgroups,
                        o_duploffs, o_ready, o_rowsrc, ntiles, o_slotflag, o_srcinfo, o_push, o_pushw, gcap, lcap, chunk)
