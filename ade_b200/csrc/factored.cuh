// Factored application  out = base_term + U^ (V^T x)  for T <= 128 tokens, one launch.
//
// Replaces the reference's decode kernels A and B and the cuBLAS call in front of them
// (src/kernels.py:486-886, src/serving.py:106).  One persistent grid (one CTA per SM) does, per CTA:
//
//   phase A  (a few CTAs)  h[t][k] = sum_n bf16((Vcode[k][n] - vz[g][n]) * vs[g][n]) * x[t][n] for 16 ranks k,
//                          written to global scratch as bf16, then one release-increment of a counter;
//   phase W  (all CTAs)    y[t][m] = sum_n w_b[m][n] x[t][n] for this CTA's contiguous slice of rows m,
//                          kept in shared memory (skipped when the caller supplies y_dense);
//   wait                   until the counter shows that every h unit has been written (bounded spin);
//   phase U  (all CTAs)    out[t][m] = y[t][m] + sum_g us[m][g] * sum_{k in g} (Ucode[m][k] - uz[m][g]) * h[t][k].
//
// Phase A is 3 % of the bytes but a full memory round trip under load.  For T <= 16 four extra warps
// per CTA run it next to the eight that stream W_b (a unit is then 16 ranks x half of d_i, written as a
// float32 partial sum; the halves are added and rounded to bf16 once per CTA, into shared memory, before
// phase U), so the grid-wide dependency h -> phase U costs no idle time.  For larger T the main warps
// run phase A first and the CTAs that own a unit get fewer rows.  Rows are otherwise split evenly over
// the CTAs (to within one row), so every SM streams the same number of bytes of W_b.
//
// All three phases are weight-streaming skinny GEMMs: the weights (bf16 rows of W_b, or 4-bit codes)
// are the 16-row operand of a warp MMA; the activations (x or h, L1/L2 resident) are the 8-column operand.
// Two variants of the W_b stream: 128-bit loads into registers two or three blocks ahead of their use, or
// (FIFO = true: up to 8 tokens, and up to 16 for long streams) per-thread cp.async copies into a FIFO in
// shared memory (as many stages as fit, three at present), with the side warps staging their operands a wave at
// a time.
// The contraction axis is split over the 8 warps of a CTA and reduced through shared memory in a
// fixed order, so results do not depend on scheduling (no floating-point atomics).
//
// Fragment bookkeeping (mma.m16n8k16, lane = 4*gid + tig): a thread's 16-byte load covers 8 bf16 (or
// 32 codes) of one weight row; consecutive 4-element slices of it are used as the thread's k-slots
// {2tig, 2tig+1, 2tig+8, 2tig+9} of consecutive MMAs, and the activation fragment is read from the
// same 4 columns, so the products line up without any shuffle.
#pragma once
#include "ptx.cuh"

namespace ade {

constexpr int FA_WARPS = 8;
constexpr int FA_THREADS = FA_WARPS * 32;
constexpr int FA_SIDE_WARPS = 4;               // extra warps that compute h = V^T x next to the W_b stream (T <= 16)
__host__ __device__ constexpr bool fa_side(int NT) { return NT <= 2; }
// Up to 8 tokens the side warps, once their share of h is written, also compute the delta term U^ h of their CTA's rows
// under the main warps' stream of W_b (measured per call on B200: q_proj T = 1 11.4 -> 10.2 us, gate_proj 25.6 -> 22.7,
// down_proj 21.1 -> 19.9).  At 9-16 tokens four warps take longer over phase U than the stream lasts (gate_proj T = 16
// 31.0 -> 34.3 us, also with their operands loaded an item ahead), so there the main warps do it after their stream, as
// above 16 tokens.
__host__ __device__ constexpr bool fa_side_u(int NT) { return NT == 1; }
__host__ __device__ constexpr int fa_threads(int NT) { return FA_THREADS + (fa_side(NT) ? FA_SIDE_WARPS * 32 : 0); }

// barrier among the 8 main warps only (the side warps never join it)
__device__ __forceinline__ void main_sync() { asm volatile("bar.sync 1, %0;" ::"n"(FA_THREADS) : "memory"); }
__device__ __forceinline__ void side_sync() { asm volatile("bar.sync 2, %0;" ::"n"(FA_SIDE_WARPS * 32) : "memory"); }
constexpr int FA_ROWS = 32;                    // output rows per pass (two m16 tiles per warp)
constexpr uint32_t kBf2_128 = 0x43004300u;     // bf16x2 (128, 128)
constexpr long long FA_SPIN_LIMIT = 2000000000LL;   // default limit of a grid-wide wait in clock cycles (about one second)

struct FactoredParams {
    const __nv_bfloat16* w_b;      // [M][N] or nullptr
    const __nv_bfloat16* x;        // [T][N]
    const __nv_bfloat16* y_dense;  // [T][M] or nullptr
    const uint8_t* uq;             // [M][r/2]
    const uint8_t* vt;             // [r][N/2]
    const uint16_t* us;            // [M][ng]
    const uint8_t* uz;             // [M][ng]
    const uint16_t* vs;            // [ng][N]
    const uint8_t* vz;             // [ng][N]
    __nv_bfloat16* h;              // scratch: bf16 [T][r], or float32 [2][T][r] partial sums when T <= 16
    float* hpart;                  // scratch, T > 16 and parts > 1: float32 [parts][T][r] partial sums of h
    int parts;                     // T > 16: every 16-rank unit of phase A is split over this many slices of d_i
    unsigned int* sync;            // scratch: [0] units arrived, [1] CTAs done, [2] status (0 = ok), [3] slices of h reduced
    unsigned int* status;          // where an expired wait records 1: sync + 2, or a word that outlives the call's memset
    long long spin_limit;          // clock cycles after which a grid-wide wait gives up
    int drop_arrivals;             // diagnostic: phase-A units do not report, so that the wait for h runs out
    __nv_bfloat16* out;            // [T][M]
    int T, M, N, r;
    int rows_cap;                  // rows of the y buffer in shared memory (multiple of 32)
    int unit_rows;                 // rows a CTA gives up for the phase-A unit it owns
    int stages;                    // depth of the shared-memory FIFO that streams W_b (0: register prefetch)
    int upf;                       // phase-U items per warp whose operands are prefetched into shared memory (0..FA_UPF)
    int hstage;                    // T > 16: h (bf16 [T][r]) is copied to shared memory before phase U (when it fits)
    int n_blocks;                  // block-diagonal U^: rows [block_rows[i], block_rows[i+1]) use groups
    int block_rows[5];             // [block_groups[i], block_groups[i+1]) only; 0 blocks = dense
    int block_groups[5];
};

// Rank groups that rows [blk, blk_end) can touch (union over the blocks they overlap).
__device__ __forceinline__ void fa_group_range(const FactoredParams& p, int blk, int blk_end, int& g_lo, int& g_hi) {
    g_lo = 0;
    g_hi = p.r >> 7;
    if (p.n_blocks > 0) {
        int lo = g_hi, hi = 0;
        for (int i = 0; i < p.n_blocks; ++i)
            if (p.block_rows[i] < blk_end && p.block_rows[i + 1] > blk) {
                lo = min(lo, p.block_groups[i]);
                hi = max(hi, p.block_groups[i + 1]);
            }
        if (hi > lo) {
            g_lo = lo;
            g_hi = hi;
        }
    }
}

// Side warps stage the V codes, scales and zero-points of up to FA_STAGE_CHUNKS chunks of 128 columns per warp
// (16 ranks x 64 bytes of codes, 256 bytes of scales, 128 bytes of zero-points per chunk) with cp.async, so that
// a whole wave of chunks is one memory round trip.  The region is reused for h (bf16 [T][r + 8]) in phase U.
constexpr int FA_STAGE_CHUNKS = 4;
constexpr int FA_STAGE_CHUNK_BYTES = 16 * 64 + 256 + 128;
__host__ __device__ constexpr size_t fa_side_region(int T, int r) {
    const size_t hs = static_cast<size_t>(T) * (r + 8) * 2 + 16;
    const size_t st = static_cast<size_t>(FA_SIDE_WARPS) * FA_STAGE_CHUNKS * FA_STAGE_CHUNK_BYTES;
    return hs > st ? hs : st;
}
// one FIFO item = one 64-column block of 32 rows of W_b (8 x 16 bytes per main thread) and the matching
// activations (2 x 16 bytes per 8 tokens)
__host__ __device__ constexpr int fa_fifo_item(int NT) { return (8 + 2 * NT) * 16 * FA_THREADS; }
constexpr int FA_FIFO_MAX = 5;

// without the FIFO; the launch adds stages * fa_fifo_item(NT) in front
// With side warps (T <= 16) the side team has a reduction buffer of its own; up to 8 tokens, where it also computes the
// delta term U^ h of the CTA's rows while the main warps still stream W_b, that buffer is [4][32][33] and there is a
// second row buffer for the delta term.
__host__ __device__ constexpr int fa_side_red_floats(int NT) { return fa_side(NT) ? FA_SIDE_WARPS * 32 * (fa_side_u(NT) ? 33 : 17) : 0; }
__host__ __device__ inline size_t factored_smem_bytes(int NT, int rows_cap, int T, int r) {
    return (static_cast<size_t>(FA_WARPS) * 32 * 33 + fa_side_red_floats(NT) +
            static_cast<size_t>(rows_cap) * (8 * NT + 1) * (fa_side_u(NT) ? 2 : 1)) * sizeof(float) +
           (fa_side(NT) ? fa_side_region(T, r) : 0);
}

// one packed word (8 codes) -> 4 bf16x2 registers holding 128 + code, codes in natural order
__device__ __forceinline__ void unpack8_bf16(uint32_t w, uint32_t (&e)[4]) {
    e[0] = (w & 0x000F000Fu) | kBf2_128;
    e[1] = ((w >> 4) & 0x000F000Fu) | kBf2_128;
    e[2] = ((w >> 8) & 0x000F000Fu) | kBf2_128;
    e[3] = ((w >> 12) & 0x000F000Fu) | kBf2_128;
}

__device__ __forceinline__ void fa_cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void fa_cp_async16_zfill(uint32_t dst_smem, const void* src, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void fa_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void fa_cp_async_wait(int n) {      // at most n of this thread's groups still in flight
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    }
}

// Sum a team's partial tiles in a fixed order (TEAM = 8: the main warps, 4: the side warps).  acc[mt][nt][4] covers
// 32 rows x 8*NT tokens; sink(row, token, sum) is called once per element by exactly one thread of the team.
template <int TEAM>
__device__ __forceinline__ void team_sync() {
    if (TEAM == FA_WARPS) main_sync(); else side_sync();
}
template <int NT, int TEAM, class Sink>
__device__ __forceinline__ void reduce_tiles_team(float (*red)[32][33], const float (&acc)[2][NT][4], int warp, int gid,
                                                  int tig, Sink sink) {
    const int tl = (TEAM == FA_WARPS ? threadIdx.x : threadIdx.x - FA_THREADS);      // index inside the team
#pragma unroll
    for (int b = 0; b < (NT + 3) / 4; ++b) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nt = b * 4 + j;
            if (nt < NT) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    red[warp][j * 8 + 2 * tig][mt * 16 + gid] = acc[mt][nt][0];
                    red[warp][j * 8 + 2 * tig + 1][mt * 16 + gid] = acc[mt][nt][1];
                    red[warp][j * 8 + 2 * tig][mt * 16 + gid + 8] = acc[mt][nt][2];
                    red[warp][j * 8 + 2 * tig + 1][mt * 16 + gid + 8] = acc[mt][nt][3];
                }
            }
        }
        team_sync<TEAM>();
#pragma unroll
        for (int i = 0; i < 1024 / (TEAM * 32); ++i) {
            const int e = tl + i * TEAM * 32;
            const int row = e & 31, tok = e >> 5;
            if (tok < 8 * (NT - 4 * b)) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < TEAM; ++w) s += red[w][tok][row];
                sink(row, b * 32 + tok, s);
            }
        }
        team_sync<TEAM>();
    }
}
template <int NT, class Sink>
__device__ __forceinline__ void reduce_tiles(float (*red)[32][33], const float (&acc)[2][NT][4], int warp, int gid,
                                             int tig, Sink sink) {
    reduce_tiles_team<NT, FA_WARPS>(red, acc, warp, gid, tig, sink);
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[2][NT][4]) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
}

// ---------------------------------------------------------------------------------------------
// phase A: h for the 16 ranks k0 .. k0+15; the d_i axis is split over the warps in chunks of 128.
// ---------------------------------------------------------------------------------------------
template <int NT>
struct XvRegs {
    uint4 q0, q1;              // 32 codes of ranks gid and gid + 8
    uint4 s[4];                // 32 bf16 scales of the thread's columns
    uint4 z[2];                // 32 zero-points
    uint4 x[NT <= 2 ? NT : 1][4];   // activations of the thread's columns (prefetched only for small T)
};

template <int NT>
__device__ __forceinline__ void xv_load(XvRegs<NT>& R, const FactoredParams& p, const uint8_t* row0,
                                        const uint8_t* row1, int g, int nb, int gid) {
    const int N = p.N;
    R.q0 = ldg16_stream(row0 + (nb >> 1));
    R.q1 = ldg16_stream(row1 + (nb >> 1));
    const uint16_t* sp = p.vs + static_cast<size_t>(g) * N + nb;
    const uint8_t* zp = p.vz + static_cast<size_t>(g) * N + nb;
#pragma unroll
    for (int j = 0; j < 4; ++j) R.s[j] = ldg16(sp + 8 * j);
    R.z[0] = ldg16(zp);
    R.z[1] = ldg16(zp + 16);
    if (NT <= 2) {
#pragma unroll
        for (int nt = 0; nt < (NT <= 2 ? NT : 1); ++nt) {
            const int tok = min(nt * 8 + gid, p.T - 1);
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) R.x[nt][wi] = ldg16(p.x + static_cast<size_t>(tok) * N + nb + 8 * wi);
        }
    }
}

// TEAM warps (the CTA's 8 main warps, or its 4 side warps) split the d_i axis in chunks of 128 columns.
// Chunks [c_begin, c_end) only; the sum goes to hf (float32 partial, [T][r]) when given, else to p.h as bf16.
template <int NT, int TEAM, bool STAGED = false>
__device__ __forceinline__ void xv_unit(const FactoredParams& p, float* redbuf, int k0, int c_begin, int c_end,
                                        float* hf, int warp, int gid, int tig, uint8_t* stage = nullptr) {
    const int N = p.N, T = p.T;
    const int g = k0 >> 7;
    const size_t rowb = static_cast<size_t>(N >> 1);
    const uint8_t* row0 = p.vt + static_cast<size_t>(k0 + gid) * rowb;
    const uint8_t* row1 = row0 + 8 * rowb;
    float acc[2][NT][4];             // only [0] is used; [1] stays zero so that the shared reducer applies
    zero_acc<NT>(acc);
    const int nchunks = c_end;
    // one chunk of 128 columns: this thread's 32 columns of ranks gid and gid + 8 against the activations
    auto chunk_mma = [&](const uint4& q0, const uint4& q1, const uint4 (&sv)[4], const uint4 (&zv)[2],
                         const uint4 (&xv)[NT <= 2 ? NT : 1][4], int nb) {
        const uint32_t cw0[4] = {q0.x, q0.y, q0.z, q0.w};
        const uint32_t cw1[4] = {q1.x, q1.y, q1.z, q1.w};
        const uint32_t sw[16] = {sv[0].x, sv[0].y, sv[0].z, sv[0].w, sv[1].x, sv[1].y, sv[1].z, sv[1].w,
                                 sv[2].x, sv[2].y, sv[2].z, sv[2].w, sv[3].x, sv[3].y, sv[3].z, sv[3].w};
        const uint32_t zw[8] = {zv[0].x, zv[0].y, zv[0].z, zv[0].w, zv[1].x, zv[1].y, zv[1].z, zv[1].w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {                  // 8 columns per packed word
            uint32_t e0[4], e1[4], a0[4], a1[4];
            unpack8_bf16(cw0[wi], e0);
            unpack8_bf16(cw1[wi], e1);
            const uint32_t zz[4] = {__byte_perm(zw[2 * wi], 0x43434343u, 0x4140),
                                    __byte_perm(zw[2 * wi], 0x43434343u, 0x4342),
                                    __byte_perm(zw[2 * wi + 1], 0x43434343u, 0x4140),
                                    __byte_perm(zw[2 * wi + 1], 0x43434343u, 0x4342)};
#pragma unroll
            for (int q = 0; q < 4; ++q) {                 // (code - zero) is exact; one rounding in the product
                a0[q] = bf2_mul(bf2_sub(e0[q], zz[q]), sw[4 * wi + q]);
                a1[q] = bf2_mul(bf2_sub(e1[q], zz[q]), sw[4 * wi + q]);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + gid;
                uint4 xq;
                if (NT <= 2) xq = xv[NT <= 2 ? nt : 0][wi];
                else xq = ldg16(p.x + static_cast<size_t>(min(tok, T - 1)) * N + nb + 8 * wi);
                if (tok >= T) xq = make_uint4(0u, 0u, 0u, 0u);
                mma_bf16(acc[0][nt], a0[0], a1[0], a0[1], a1[1], xq.x, xq.y);
                mma_bf16(acc[0][nt], a0[2], a1[2], a0[3], a1[3], xq.z, xq.w);
            }
        }
    };
    if constexpr (STAGED && NT <= 2) {
        // staged: every chunk of a wave is copied to shared memory at once (one round trip per wave)
        const int lane = threadIdx.x & 31;
        uint8_t* mine = stage + static_cast<size_t>(warp) * (FA_STAGE_CHUNKS * FA_STAGE_CHUNK_BYTES);
        const uint32_t mine_s = smem_u32(mine);
        auto load_x = [&](uint4 (&xv)[NT <= 2 ? NT : 1][4], int nb) {
#pragma unroll
            for (int nt = 0; nt < (NT <= 2 ? NT : 1); ++nt) {
                const int tok = min(nt * 8 + gid, T - 1);
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) xv[nt][wi] = ldg16(p.x + static_cast<size_t>(tok) * N + nb + 8 * wi);
            }
        };
        // chunks per wave: as many as the staging area holds, but the activations of a whole wave sit in registers
        // (they are plain loads: issued late they would queue behind the copy stream of the main warps)
        constexpr int CH = NT == 1 ? FA_STAGE_CHUNKS : FA_STAGE_CHUNKS / 2;
        for (int cw = c_begin + warp; cw < nchunks; cw += TEAM * CH) {
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int c = cw + k * TEAM;
                if (c < nchunks) {
                    const int cols = c << 7;
                    const uint32_t dst = mine_s + k * FA_STAGE_CHUNK_BYTES;
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int pid = lane + 32 * h2;   // 16 ranks x 4 pieces of 16 bytes
                        fa_cp_async16(dst + pid * 16, p.vt + static_cast<size_t>(k0 + (pid >> 2)) * rowb + (cols >> 1) + (pid & 3) * 16);
                    }
                    if (lane < 16) fa_cp_async16(dst + 1024 + lane * 16, p.vs + static_cast<size_t>(g) * N + cols + 8 * lane);
                    else if (lane < 24) fa_cp_async16(dst + 1280 + (lane - 16) * 16, p.vz + static_cast<size_t>(g) * N + cols + 16 * (lane - 16));
                }
            }
            fa_cp_async_commit();
            uint4 xw[CH][NT <= 2 ? NT : 1][4];
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int c = min(cw + k * TEAM, nchunks - 1);
                load_x(xw[k], (c << 7) + tig * 32);
            }
            fa_cp_async_wait(0);
            __syncwarp();
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int c = cw + k * TEAM;
                if (c < nchunks) {
                    const int nb = (c << 7) + tig * 32;
                    const uint8_t* src = mine + k * FA_STAGE_CHUNK_BYTES;
                    const uint4 q0 = *reinterpret_cast<const uint4*>(src + gid * 64 + tig * 16);
                    const uint4 q1 = *reinterpret_cast<const uint4*>(src + (gid + 8) * 64 + tig * 16);
                    uint4 sv[4], zv[2];
#pragma unroll
                    for (int j = 0; j < 4; ++j) sv[j] = *reinterpret_cast<const uint4*>(src + 1024 + tig * 64 + j * 16);
                    zv[0] = *reinterpret_cast<const uint4*>(src + 1280 + tig * 32);
                    zv[1] = *reinterpret_cast<const uint4*>(src + 1280 + tig * 32 + 16);
                    chunk_mma(q0, q1, sv, zv, xw[k], nb);
                }
            }
            __syncwarp();                                  // the next wave overwrites the staging area
        }
    } else {
        XvRegs<NT> cur, nxt;             // one chunk in flight while the previous one is multiplied
        if (c_begin + warp < nchunks) xv_load<NT>(cur, p, row0, row1, g, ((c_begin + warp) << 7) + tig * 32, gid);
        for (int c = c_begin + warp; c < nchunks; c += TEAM) {
            const int nb = (c << 7) + tig * 32;               // this thread's 32 columns
            if (c + TEAM < nchunks) xv_load<NT>(nxt, p, row0, row1, g, ((c + TEAM) << 7) + tig * 32, gid);
            chunk_mma(cur.q0, cur.q1, cur.s, cur.z, cur.x, nb);
            if (c + TEAM < nchunks) cur = nxt;
        }
    }
    // fixed-order sum over the team, 32 tokens at a time: redbuf[TEAM][32 tokens][16 ranks (+1 pad)]
    float (*red)[32][17] = reinterpret_cast<float (*)[32][17]>(redbuf);
    const int tl = (TEAM == FA_WARPS ? threadIdx.x : threadIdx.x - FA_THREADS);      // index inside the team
#pragma unroll
    for (int b = 0; b < (NT + 3) / 4; ++b) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nt = b * 4 + j;
            if (nt < NT) {
                red[warp][j * 8 + 2 * tig][gid] = acc[0][nt][0];
                red[warp][j * 8 + 2 * tig + 1][gid] = acc[0][nt][1];
                red[warp][j * 8 + 2 * tig][gid + 8] = acc[0][nt][2];
                red[warp][j * 8 + 2 * tig + 1][gid + 8] = acc[0][nt][3];
            }
        }
        if (TEAM == FA_WARPS) main_sync(); else side_sync();
        for (int e = tl; e < 16 * 32; e += TEAM * 32) {
            const int rank = e & 15, tok = e >> 4;
            const int t = b * 32 + tok;
            if (tok < 8 * (NT - 4 * b) && t < T) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < TEAM; ++w) sum += red[w][tok][rank];
                if (hf) hf[static_cast<size_t>(t) * p.r + k0 + rank] = sum;
                else p.h[static_cast<size_t>(t) * p.r + k0 + rank] = __float2bfloat16_rn(sum);
            }
        }
        if (TEAM == FA_WARPS) main_sync(); else side_sync();
    }
}

// ---------------------------------------------------------------------------------------------
// phase W: acc += W_b[rows] x^T over this warp's share of the d_i axis (blocks of 64 columns,
// block b -> warp b % 8), weights and activations loaded DEPTH-1 blocks ahead.
// Every CTA starts at another block (rotation by blockIdx.x): all CTAs read the same few kilobytes of x, and walking
// them in step made every SM ask L2 for the same lines at the same time (measured: 4-6 % per call at T >= 4).
// ---------------------------------------------------------------------------------------------
template <int NT, int DEPTH, bool PREFETCH_X>
__device__ __forceinline__ void wx_block(const FactoredParams& p, float (&acc)[2][NT][4], int blk, int row_end,
                                         int warp, int gid, int tig) {
    const int N = p.N, T = p.T;
    const int nblk = N >> 6;
    const int cnt = (nblk - warp + FA_WARPS - 1) / FA_WARPS;        // blocks of this warp
    const __nv_bfloat16* wrow[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            // rows past the slice re-read the last one (L1 / L2 hits); predicating them off was measured slower
            const int m = min(blk + mt * 16 + hr * 8 + gid, row_end - 1);
            wrow[mt][hr] = p.w_b + static_cast<size_t>(m) * N + tig * 8;
        }
    const __nv_bfloat16* xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xrow[nt] = p.x + static_cast<size_t>(min(nt * 8 + gid, T - 1)) * N + tig * 8;

    uint4 A[DEPTH][2][2][2];
    uint4 X[PREFETCH_X ? DEPTH : 1][NT][2];
    auto load = [&](int d, int i) {
        const int col = (warp + FA_WARPS * ((i + static_cast<int>(blockIdx.x)) % cnt)) * 64;   // see wx_block's note on the rotation
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int hr = 0; hr < 2; ++hr)
#pragma unroll
                for (int s = 0; s < 2; ++s) A[d][mt][hr][s] = ldg16_stream(wrow[mt][hr] + col + s * 32);
        if (PREFETCH_X) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int s = 0; s < 2; ++s) X[d][nt][s] = ldg16(xrow[nt] + col + s * 32);
        }
    };
    auto compute = [&](int d, int i) {
        const int col = (warp + FA_WARPS * ((i + static_cast<int>(blockIdx.x)) % cnt)) * 64;   // see wx_block's note on the rotation
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const bool live = nt * 8 + gid < T;
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                uint4 xq = PREFETCH_X ? X[d][nt][s] : ldg16(xrow[nt] + col + s * 32);
                if (!live) xq = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma_bf16(acc[mt][nt], A[d][mt][0][s].x, A[d][mt][1][s].x, A[d][mt][0][s].y, A[d][mt][1][s].y,
                             xq.x, xq.y);
                    mma_bf16(acc[mt][nt], A[d][mt][0][s].z, A[d][mt][1][s].z, A[d][mt][0][s].w, A[d][mt][1][s].w,
                             xq.z, xq.w);
                }
            }
        }
    };
#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d)
        if (d < cnt) load(d, d);
    for (int i = 0; i < cnt; i += DEPTH) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int ii = i + d;
            if (ii < cnt) {
                if (ii + DEPTH - 1 < cnt) load((d + DEPTH - 1) % DEPTH, ii + DEPTH - 1);
                compute(d, ii);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// phase W through a shared-memory FIFO: the same 16-byte pieces as wx_block, but every thread copies
// its own pieces with cp.async `stages - 1` blocks ahead (across the CTA's row blocks), so that
// several items per thread are in flight without holding them in registers (x included: a plain load of x
// would queue behind the copies and pay the loaded memory latency every item).  A thread reads back only what
// it copied itself: no barrier guards the FIFO.  y goes to ybuf[row - row0][token].
// ---------------------------------------------------------------------------------------------
template <int NT>
__device__ __forceinline__ void wx_stream(const FactoredParams& p, float (*red)[32][33], float* ybuf, const uint8_t* fifo,
                                          int row0, int row1, int warp, int gid, int tig) {
    constexpr int YS = 8 * NT + 1;
    constexpr uint32_t STR = FA_THREADS * 16;               // distance between a thread's pieces of one item
    constexpr int ITEM = fa_fifo_item(NT);
    const int N = p.N, T = p.T, S = p.stages;
    const int nblk = N >> 6;
    const int cnt = (nblk - warp + FA_WARPS - 1) / FA_WARPS;        // 64-column blocks of this warp per row block
    const int nb = (row1 - row0 + FA_ROWS - 1) / FA_ROWS;
    const int total = nb * cnt;
    const uint32_t fs = smem_u32(fifo) + threadIdx.x * 16;
    const uint4* fr = reinterpret_cast<const uint4*>(fifo) + threadIdx.x;
    const __nv_bfloat16* xrow[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xrow[nt] = p.x + static_cast<size_t>(min(nt * 8 + gid, T - 1)) * N + tig * 8;

    int qi = 0, qb = 0;                                     // block column index and row block of the next item to issue
    auto issue = [&](int q) {
        if (q < total) {
            const uint32_t sb = fs + (q % S) * ITEM;
            const int col = (warp + FA_WARPS * ((qi + static_cast<int>(blockIdx.x)) % cnt)) * 64 + tig * 8;   // rotated as in wx_block
            const int blk = row0 + qb * FA_ROWS;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                // the slice's last block may hold 16 rows or fewer (5120 rows over 148 CTAs are 34.6 each): its second
                // m16 tile is then neither copied nor multiplied (skipping single eight-row halves as well was slower)
                if (mt == 1 && blk + 16 >= row1) break;
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    const int m = min(blk + mt * 16 + hr * 8 + gid, row1 - 1);     // rows past the slice: re-read the last one
                    const __nv_bfloat16* src = p.w_b + static_cast<size_t>(m) * N + col;
                    fa_cp_async16(sb + (mt * 4 + hr * 2) * STR, src);
                    fa_cp_async16(sb + (mt * 4 + hr * 2 + 1) * STR, src + 32);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // lanes whose token does not exist copy nothing (zero fill): eight lanes asking for the same
                // 16 bytes of the last token made the stream measurably slower at T = 1 than at T = 8
                const bool lv = nt * 8 + gid < T;
                fa_cp_async16_zfill(sb + (8 + 2 * nt) * STR, xrow[nt] + col - tig * 8, lv);
                fa_cp_async16_zfill(sb + (9 + 2 * nt) * STR, xrow[nt] + col - tig * 8 + 32, lv);
            }
            if (++qi == cnt) {
                qi = 0;
                ++qb;
            }
        }
        fa_cp_async_commit();                              // one group per call, empty past the end
    };
    for (int q = 0; q < S - 1; ++q) issue(q);

    int q = 0;
    for (int b = 0; b < nb; ++b) {
        float acc[2][NT][4];
        zero_acc<NT>(acc);
        const bool tile1 = row0 + b * FA_ROWS + 16 < row1;  // the block's second m16 tile holds rows of the slice
        for (int i = 0; i < cnt; ++i, ++q) {
            fa_cp_async_wait(S - 2);                        // item q has landed
            uint4 A[2][2][2];
            const uint4* slot = fr + static_cast<size_t>(q % S) * (ITEM / 16);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr)
#pragma unroll
                    for (int s2 = 0; s2 < 2; ++s2)
                        A[mt][hr][s2] = (mt == 0 || tile1) ? slot[(mt * 4 + hr * 2 + s2) * FA_THREADS] : make_uint4(0u, 0u, 0u, 0u);
            uint4 X[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2) X[nt][s2] = slot[(8 + 2 * nt + s2) * FA_THREADS];
            issue(q + S - 1);                               // refills the slot read one iteration ago
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const bool live = nt * 8 + gid < T;
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2) {
                    uint4 xq = X[nt][s2];
                    if (!live) xq = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        if (mt == 1 && !tile1) break;
                        mma_bf16(acc[mt][nt], A[mt][0][s2].x, A[mt][1][s2].x, A[mt][0][s2].y, A[mt][1][s2].y, xq.x, xq.y);
                        mma_bf16(acc[mt][nt], A[mt][0][s2].z, A[mt][1][s2].z, A[mt][0][s2].w, A[mt][1][s2].w, xq.z, xq.w);
                    }
                }
            }
        }
        float* yb = ybuf + static_cast<size_t>(b) * FA_ROWS * YS;
        reduce_tiles<NT>(red, acc, warp, gid, tig, [=](int row, int t, float s) { yb[row * YS + t] = s; });
    }
    fa_cp_async_wait(0);
}

// ---------------------------------------------------------------------------------------------
// phase U: acc += sum_g us * (Ucode - uz)[rows, group g] h^T.  A work item is one m16 tile of the 32-row block
// times one rank group; item j = 2 g + tile goes to warp j % 8, so four warps already share a block at r = 256.
// The operands of a warp's first FA_UPF items (over all its row blocks) are copied to shared memory before the
// grid-wide wait for h (they do not depend on it), which takes their memory round trip off the path behind it.
// ---------------------------------------------------------------------------------------------
constexpr int FA_UPF = 4;
// phase-U work items per (m16 tile, rank group): the token tiles are shared out as well when there are many, so that
// all eight warps have work at small ranks
__host__ __device__ constexpr int fa_u_split(int NT) { return NT >= 16 ? 4 : (NT >= 8 ? 2 : 1); }
constexpr int FA_UPF_ITEM = FA_THREADS * (2 * 16 + 2 * 8);     // per item and thread: two 16-byte code pieces, two (zero, scale) word pairs
__device__ __forceinline__ void fa_cp_async4(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}

__device__ __forceinline__ void uh_prefetch(const FactoredParams& p, uint8_t* ustage, int row0, int row1, int warp, int gid,
                                            int tig, int ns) {
    const int ng = p.r >> 7;
    const size_t rowb = static_cast<size_t>(p.r >> 1);
    const uint32_t us_s = smem_u32(ustage);
    int k = 0;
    for (int blk = row0; blk < row1 && k < p.upf; blk += FA_ROWS) {
        int g_lo, g_hi;
        fa_group_range(p, blk, min(blk + FA_ROWS, row1), g_lo, g_hi);
        for (int j = warp; j < 2 * (g_hi - g_lo) * ns && k < p.upf; j += FA_WARPS, ++k) {
            const int jj = j / ns, mt = jj & 1, g = g_lo + (jj >> 1);
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int m = min(blk + mt * 16 + hr * 8 + gid, row1 - 1);
                const size_t e = static_cast<size_t>(m) * ng + g;
                const uint32_t base = us_s + k * FA_UPF_ITEM;
                fa_cp_async16(base + (hr * FA_THREADS + threadIdx.x) * 16, p.uq + static_cast<size_t>(m) * rowb + g * 64 + tig * 16);
                const uint32_t sc = base + 2 * FA_THREADS * 16 + (hr * FA_THREADS + threadIdx.x) * 8;
                fa_cp_async4(sc, p.uz + (e & ~static_cast<size_t>(3)));                 // the aligned word that holds the zero-point
                fa_cp_async4(sc + 4, p.us + (e & ~static_cast<size_t>(1)));             // ... and the one that holds the scale
            }
        }
    }
    fa_cp_async_commit();
}

// Operands of one phase-U work item as a thread holds them: 32 codes of rows gid and gid + 8 of an m16 tile, and the
// zero-point and scale of those rows for the item's rank group.
struct UOperand {
    uint4 q[2];
    uint32_t z[2], s[2];
};
__device__ __forceinline__ void uh_fetch(const FactoredParams& p, UOperand& o, int blk, int row_end, int mt, int g, int gid, int tig) {
    const int ng = p.r >> 7;
    const size_t rowb = static_cast<size_t>(p.r >> 1);
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        const int m = min(blk + mt * 16 + hr * 8 + gid, row_end - 1);
        const size_t e = static_cast<size_t>(m) * ng + g;
        o.q[hr] = ldg16_stream(p.uq + static_cast<size_t>(m) * rowb + g * 64 + tig * 16);
        o.z[hr] = p.uz[e];
        o.s[hr] = p.us[e];
    }
}
// acc += us * (Ucode - uz)[m16 tile mt, group g] h^T for the token tiles of `part`
template <int NT, bool SPLIT>
__device__ __forceinline__ void uh_compute(const FactoredParams& p, float (&acc)[2][NT][4], const UOperand& o, int mt, int g, int part,
                                           const __nv_bfloat16* hs, int gid, int tig) {
    constexpr int NS = fa_u_split(NT);
    const int T = p.T, r = p.r;
    uint32_t a[2][16];           // [row gid / gid+8][pair]: (code - zero) as bf16x2
    float su[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        const uint32_t zz = kBf2_128 | o.z[hr] | (o.z[hr] << 16);
        su[hr] = bf16_bits_to_f32(static_cast<uint16_t>(o.s[hr]));
        const uint32_t cw[4] = {o.q[hr].x, o.q[hr].y, o.q[hr].z, o.q[hr].w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            uint32_t ev[4];
            unpack8_bf16(cw[wi], ev);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) a[hr][4 * wi + q4] = bf2_sub(ev[q4], zz);
        }
    }
    const int kb = g * 128 + tig * 32;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        if (NS > 1 && nt / (NT / NS) != part) continue;
        const int tok = nt * 8 + gid;
        float pa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            uint4 hq = make_uint4(0u, 0u, 0u, 0u);
            if (tok < T) {
                if (SPLIT || hs != nullptr) hq = *reinterpret_cast<const uint4*>(hs + static_cast<size_t>(tok) * (r + 8) + kb + 8 * wi);
                else hq = ldcg16(p.h + static_cast<size_t>(tok) * r + kb + 8 * wi);
            }
            mma_bf16(pa, a[0][4 * wi], a[1][4 * wi], a[0][4 * wi + 1], a[1][4 * wi + 1], hq.x, hq.y);
            mma_bf16(pa, a[0][4 * wi + 2], a[1][4 * wi + 2], a[0][4 * wi + 3], a[1][4 * wi + 3], hq.z, hq.w);
        }
        // one rescale per group; mt selects the accumulator tile
        if (mt == 0) {
            acc[0][nt][0] += su[0] * pa[0];
            acc[0][nt][1] += su[0] * pa[1];
            acc[0][nt][2] += su[1] * pa[2];
            acc[0][nt][3] += su[1] * pa[3];
        } else {
            acc[1][nt][0] += su[0] * pa[0];
            acc[1][nt][1] += su[0] * pa[1];
            acc[1][nt][2] += su[1] * pa[2];
            acc[1][nt][3] += su[1] * pa[3];
        }
    }
}

// SPLIT: h has been staged in shared memory (hs, bf16 [T][r + 8]); otherwise it is read from p.h (L2).
// k: running index of this warp's items over the blocks (the first p.upf were prefetched into shared memory before the
// grid-wide wait; the others are loaded one item ahead of their use).
template <int NT, bool SPLIT, int TEAM = FA_WARPS>
__device__ __forceinline__ void uh_block(const FactoredParams& p, float (&acc)[2][NT][4], int blk, int row_end,
                                         const __nv_bfloat16* hs, const uint8_t* ustage, int& k, int warp, int gid, int tig) {
    const int ng = p.r >> 7;
    int g_lo, g_hi;
    fa_group_range(p, blk, min(blk + FA_ROWS, row_end), g_lo, g_hi);
    constexpr int NS = fa_u_split(NT);
    const int n = 2 * (g_hi - g_lo) * NS;
    UOperand cur, nxt;
    if (warp < n && k >= p.upf) uh_fetch(p, cur, blk, row_end, (warp / NS) & 1, g_lo + ((warp / NS) >> 1), gid, tig);
    for (int j = warp; j < n; j += TEAM, ++k) {
        const int part = j % NS, jj = j / NS;               // token tiles [part * NT / NS, (part + 1) * NT / NS)
        const int mt = jj & 1, g = g_lo + (jj >> 1);
        const int jn = j + TEAM;
        if (jn < n && k + 1 >= p.upf) uh_fetch(p, nxt, blk, row_end, (jn / NS) & 1, g_lo + ((jn / NS) >> 1), gid, tig);
        if (k < p.upf) {
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int m = min(blk + mt * 16 + hr * 8 + gid, row_end - 1);
                const size_t e = static_cast<size_t>(m) * ng + g;
                const uint8_t* base = ustage + static_cast<size_t>(k) * FA_UPF_ITEM;
                cur.q[hr] = *reinterpret_cast<const uint4*>(base + (hr * FA_THREADS + threadIdx.x) * 16);
                const uint2 w = *reinterpret_cast<const uint2*>(base + 2 * FA_THREADS * 16 + (hr * FA_THREADS + threadIdx.x) * 8);
                cur.z[hr] = (w.x >> (8 * static_cast<uint32_t>(e & 3))) & 0xFFu;
                cur.s[hr] = (w.y >> (16 * static_cast<uint32_t>(e & 1))) & 0xFFFFu;
            }
        }
        uh_compute<NT, SPLIT>(p, acc, cur, mt, g, part, hs, gid, tig);
        cur = nxt;
    }
}

// First row of CTA c's slice.  The last `unit_ctas` CTAs own a phase-A unit each and give up
// `unit_rows` rows for it; the rows are otherwise split evenly.
__device__ __forceinline__ int slice_start(int c, int G, int M, int unit_ctas, int unit_rows) {
    if (c >= G) return M;
    const long long budget = static_cast<long long>(M) + static_cast<long long>(unit_ctas) * unit_rows;
    long long s = budget * c / G;
    const int first = G - unit_ctas;
    if (c > first) s -= static_cast<long long>(c - first) * unit_rows;
    return static_cast<int>(s < 0 ? 0 : (s > M ? M : s));
}

// FIFO: W_b streams through the shared-memory FIFO and the side warps stage their operands (T <= 16 and a
// base weight only); a separate instantiation, so that the register-prefetch variant keeps its registers.
template <int NT, bool FUSE_WB, bool FIFO = false>
__global__ void __launch_bounds__(fa_threads(NT)) factored_kernel(const FactoredParams p) {
    extern __shared__ float fsmem_all[];
    const uint8_t* fifo = reinterpret_cast<const uint8_t*>(fsmem_all);                  // [stages][fa_fifo_item(NT)], may be empty
    float* fsmem = fsmem_all + static_cast<size_t>(p.stages) * (fa_fifo_item(NT) / 4);
    float (*red)[32][33] = reinterpret_cast<float (*)[32][33]>(fsmem);
    constexpr int YS = 8 * NT + 1;                         // padded row stride of the y buffer
    constexpr bool SIDE = fa_side(NT);
    constexpr bool SIDE_U = fa_side_u(NT);                 // the side warps also compute the delta term (phase U)
    float* side_red = fsmem + FA_WARPS * 32 * 33;          // the side team's reduction buffer
    float* ybuf = side_red + fa_side_red_floats(NT);       // [rows_cap][YS] base term of the CTA's rows
    float* ydel = ybuf + static_cast<size_t>(p.rows_cap) * YS;         // [rows_cap][YS] delta term (SIDE_U only)
    float* after_rows = ybuf + static_cast<size_t>(p.rows_cap) * YS * (SIDE_U ? 2 : 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int G = gridDim.x, c = blockIdx.x;
    const int parts = SIDE ? 2 : p.parts;                  // slices of d_i per 16 ranks (side warps: two halves)
    const int n_units = (p.r >> 4) * parts;
    const int unit_ctas = min(n_units, G);
    const int nchunks = p.N >> 7;
    const int row0 = slice_start(c, G, p.M, unit_ctas, p.unit_rows);
    const int row1 = slice_start(c + 1, G, p.M, unit_ctas, p.unit_rows);

    // ---- phase A: units are dealt from the last CTA backwards.  With side warps (T <= 16) they do it
    // while the main warps are already streaming W_b, and leave; otherwise the main warps do it first.
    if (SIDE && warp >= FA_WARPS) {
        unsigned int done = 0;
        for (int u = G - 1 - c; u < n_units; u += G) {
            const int half = u & 1, mid = (nchunks + 1) >> 1;
            xv_unit<NT, FA_SIDE_WARPS, FIFO>(p, side_red, (u >> 1) * 16, half ? mid : 0, half ? nchunks : mid,
                                       reinterpret_cast<float*>(p.h) + static_cast<size_t>(half) * p.T * p.r,
                                       warp - FA_WARPS, gid, tig,
                                       FIFO ? reinterpret_cast<uint8_t*>(after_rows) : nullptr);   // staged with the FIFO, from registers without
            ++done;
        }
        // xv_unit ended with a barrier of the side warps; the release orders their stores of h before the count.
        // One fire-and-forget instruction: a fence and an atomic would be two more memory round trips under load.
        if (done && threadIdx.x == FA_THREADS && !p.drop_arrivals) red_release_gpu_add(p.sync, done);
        if (!SIDE_U) return;

        // ---- The side warps go on to the delta term U^ h of this CTA's rows while the main warps are still streaming
        // W_b: the wait for h, the sum of its two halves, phase U and its reduction all hide under that stream, and the
        // main warps only add the two row buffers at the end.
        const int sw = warp - FA_WARPS, st = threadIdx.x - FA_THREADS;
        if (st == 0) {
            const long long t0 = clock64();
            while (ld_acquire_gpu(p.sync) < static_cast<unsigned int>(n_units)) {
                if (clock64() - t0 > p.spin_limit) {
                    atomicExch(p.status, 1u);
                    break;
                }
            }
        }
        side_sync();
        __nv_bfloat16* hs = reinterpret_cast<__nv_bfloat16*>(after_rows);    // [T][r + 8]; the staging area is free by now
        {
            // the two float32 halves of h, summed, rounded to bf16 once and kept in shared memory for phase U
            const float* h0 = reinterpret_cast<const float*>(p.h);
            const float* h1 = h0 + static_cast<size_t>(p.T) * p.r;
            const int quads = (p.T * p.r) >> 2;
            for (int i = st; i < quads; i += FA_SIDE_WARPS * 32) {
                const uint4 a = ldcg16(h0 + 4 * i), b = ldcg16(h1 + 4 * i);
                const int t = (4 * i) / p.r, k = (4 * i) % p.r;
                const __nv_bfloat162 lo = __floats2bfloat162_rn(__uint_as_float(a.x) + __uint_as_float(b.x),
                                                                __uint_as_float(a.y) + __uint_as_float(b.y));
                const __nv_bfloat162 hi = __floats2bfloat162_rn(__uint_as_float(a.z) + __uint_as_float(b.z),
                                                                __uint_as_float(a.w) + __uint_as_float(b.w));
                uint2 v;
                v.x = *reinterpret_cast<const uint32_t*>(&lo);
                v.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(hs + static_cast<size_t>(t) * (p.r + 8) + k) = v;
            }
        }
        side_sync();
        // Re-arm the counters for the next call on this scratch buffer: every CTA checks out once it is past its wait and
        // has read h; the last one to do so (nobody reads the counters or h of this call any more) zeroes them.
        if (st == 0) {
            if (atomicAdd(p.sync + 1, 1u) == static_cast<unsigned int>(G - 1)) {
                atomicExch(p.sync, 0u);
                atomicExch(p.sync + 1, 0u);
                atomicExch(p.sync + 3, 0u);
            }
        }
        float (*sred)[32][33] = reinterpret_cast<float (*)[32][33]>(side_red);
        // Phase U over the CTA's row blocks.  A warp's items are (m16 tile, rank group) pairs, item j of a block going
        // to warp j % 4; the operands of the next item, which may belong to the next block, are requested before the
        // current one is multiplied, so that their latency also hides under the reduction at the end of a block.
        auto items_of = [&](int blk, int& g_lo) {
            int g_hi;
            fa_group_range(p, blk, min(blk + FA_ROWS, row1), g_lo, g_hi);
            return 2 * (g_hi - g_lo);
        };
        UOperand cur, nxt;
        int nb = row0, nj = sw, n_glo = 0, n_n = 0;          // the next item to fetch: block, index, its block's first group and item count
        auto advance = [&]() {                                // moves (nb, nj) to the warp's next existing item, fetching it
            while (nb < row1) {
                n_n = items_of(nb, n_glo);
                if (nj < n_n) {
                    uh_fetch(p, nxt, nb, row1, nj & 1, n_glo + (nj >> 1), gid, tig);
                    return;
                }
                nb += FA_ROWS;
                nj = sw;
            }
        };
        advance();
        for (int blk = row0; blk < row1; blk += FA_ROWS) {
            float acc[2][NT][4];
            zero_acc<NT>(acc);
            while (nb == blk) {                               // every fetched item of this block
                cur = nxt;
                const int mt = nj & 1, g = n_glo + (nj >> 1);
                nj += FA_SIDE_WARPS;
                if (nj >= n_n) {
                    nb += FA_ROWS;
                    nj = sw;
                }
                advance();
                uh_compute<NT, true>(p, acc, cur, mt, g, 0, hs, gid, tig);
            }
            float* yd = ydel + static_cast<size_t>(blk - row0) * YS;
            reduce_tiles_team<NT, FA_SIDE_WARPS>(sred, acc, sw, gid, tig, [=](int row, int t, float v) { yd[row * YS + t] = v; });
        }
        asm volatile("bar.arrive 3, %0;" ::"n"(FA_THREADS + FA_SIDE_WARPS * 32) : "memory");   // the delta rows are complete
        return;
    }
    if (!SIDE) {
        unsigned int done = 0;
        for (int u = G - 1 - c; u < n_units; u += G) {
            const int part = u % parts, kb = u / parts;
            xv_unit<NT, FA_WARPS>(p, fsmem, kb * 16, part * nchunks / parts, (part + 1) * nchunks / parts,
                                  parts > 1 ? p.hpart + static_cast<size_t>(part) * p.T * p.r : nullptr, warp, gid, tig);
            ++done;
        }
        if (done && threadIdx.x == 0 && !p.drop_arrivals) {   // xv_unit ended with a barrier of the main warps
            __threadfence();
            atomicAdd(p.sync, done);
        }
    }

    // ---- phase W
    if constexpr (FIFO) {
        wx_stream<NT>(p, red, ybuf, fifo, row0, row1, warp, gid, tig);
    } else if (FUSE_WB) {
        for (int blk = row0; blk < row1; blk += FA_ROWS) {
            float acc[2][NT][4];
            zero_acc<NT>(acc);
            constexpr int DEPTH = NT == 1 ? 3 : 2;
            wx_block<NT, DEPTH, (NT <= 4)>(p, acc, blk, row1, warp, gid, tig);
            float* yb = ybuf + static_cast<size_t>(blk - row0) * YS;
            reduce_tiles<NT>(red, acc, warp, gid, tig, [=](int row, int t, float s) { yb[row * YS + t] = s; });
        }
    }

    if (!FUSE_WB) {
        // Base term supplied by the caller: this CTA's rows of y_dense go to the y buffer now, while h is still being
        // computed elsewhere, so that the store loop of phase U does not wait for a global load per element.
        const int rows = row1 - row0;
        for (int e = threadIdx.x; e < rows * p.T; e += FA_THREADS) {
            const int t = e / rows, rr = e - t * rows;
            ybuf[static_cast<size_t>(rr) * YS + t] = __bfloat162float(p.y_dense[static_cast<size_t>(t) * p.M + row0 + rr]);
        }
    }
    if constexpr (SIDE_U) {
        // The side warps have computed (or are finishing) the delta term of these rows; the output is the sum of the two
        // row buffers, one bf16 rounding.
        asm volatile("bar.sync 3, %0;" ::"n"(FA_THREADS + FA_SIDE_WARPS * 32) : "memory");
        const int rows = row1 - row0, T = p.T;
        for (int e = threadIdx.x; e < rows * T; e += FA_THREADS) {
            const int t = e / rows, rr = e - t * rows;
            p.out[static_cast<size_t>(t) * p.M + row0 + rr] =
                __float2bfloat16_rn(ydel[static_cast<size_t>(rr) * YS + t] + ybuf[static_cast<size_t>(rr) * YS + t]);
        }
        return;
    }
    // operands of the first phase-U items: in flight while this CTA waits for h.  The stream variant reuses its
    // FIFO (drained by now), the others have an area of their own behind the h tile.
    uint8_t* ustage = FIFO ? const_cast<uint8_t*>(fifo)
                           : reinterpret_cast<uint8_t*>(after_rows) + (SIDE || p.hstage ? fa_side_region(p.T, p.r) : 0);
    if (p.upf > 0) uh_prefetch(p, ustage, row0, row1, warp, gid, tig, fa_u_split(NT));

    // ---- wait for every h unit (bounded; on expiry record a status and carry on)
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        while (ld_acquire_gpu(p.sync) < static_cast<unsigned int>(n_units)) {
            if (clock64() - t0 > p.spin_limit) {
                atomicExch(p.status, 1u);
                break;
            }
        }
    }
    main_sync();
    if (!SIDE && parts > 1) {
        // The slices of d_i were summed by different CTAs: every CTA now adds the partial sums of its share of
        // the T x r elements, rounds to bf16 once and publishes them; phase U starts when all shares are there.
        const int quads = (p.T * p.r) >> 2;
        const int q0 = static_cast<int>(static_cast<long long>(c) * quads / G);
        const int q1 = static_cast<int>(static_cast<long long>(c + 1) * quads / G);
        const size_t stride = static_cast<size_t>(p.T) * p.r;
        for (int i = q0 + threadIdx.x; i < q1; i += FA_THREADS) {
            uint4 a = ldcg16(p.hpart + 4 * static_cast<size_t>(i));
            float s0 = __uint_as_float(a.x), s1 = __uint_as_float(a.y), s2 = __uint_as_float(a.z), s3 = __uint_as_float(a.w);
            for (int k = 1; k < parts; ++k) {
                a = ldcg16(p.hpart + k * stride + 4 * static_cast<size_t>(i));
                s0 += __uint_as_float(a.x);
                s1 += __uint_as_float(a.y);
                s2 += __uint_as_float(a.z);
                s3 += __uint_as_float(a.w);
            }
            const __nv_bfloat162 lo = __floats2bfloat162_rn(s0, s1), hi = __floats2bfloat162_rn(s2, s3);
            uint2 v;
            v.x = *reinterpret_cast<const uint32_t*>(&lo);
            v.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(p.h + 4 * static_cast<size_t>(i)) = v;
        }
        main_sync();
        if (threadIdx.x == 0) {
            red_release_gpu_add(p.sync + 3, 1u);
            const long long t0 = clock64();
            while (ld_acquire_gpu(p.sync + 3) < static_cast<unsigned int>(G)) {
                if (clock64() - t0 > p.spin_limit) {
                    atomicExch(p.status, 1u);
                    break;
                }
            }
        }
        main_sync();
    }
    __nv_bfloat16* hs = reinterpret_cast<__nv_bfloat16*>(after_rows);   // [T][r + 8]
    if (!SIDE) {
        if (p.hstage) {
            // h into shared memory in one sweep of 16-byte copies: phase U would otherwise fetch it from L2 in small
            // dependent loads, 64 per work item at T = 128
            const int per_row = p.r >> 3, pieces = p.T * per_row;
            const uint32_t hs_s = smem_u32(hs);
            for (int i = threadIdx.x; i < pieces; i += FA_THREADS) {
                const int t = i / per_row, k8 = i - t * per_row;
                fa_cp_async16(hs_s + (static_cast<uint32_t>(t) * (p.r + 8) + 8 * k8) * 2, p.h + static_cast<size_t>(t) * p.r + 8 * k8);
            }
            fa_cp_async_commit();
            fa_cp_async_wait(0);
            main_sync();
        } else {
            hs = nullptr;
        }
    }
    if (SIDE) {
        // the two float32 halves of h, summed, rounded to bf16 once and kept in shared memory for phase U
        const float* h0 = reinterpret_cast<const float*>(p.h);
        const float* h1 = h0 + static_cast<size_t>(p.T) * p.r;
        const int quads = (p.T * p.r) >> 2;
        for (int i = threadIdx.x; i < quads; i += FA_THREADS) {
            const uint4 a = ldcg16(h0 + 4 * i), b = ldcg16(h1 + 4 * i);
            const int t = (4 * i) / p.r, k = (4 * i) % p.r;
            const __nv_bfloat162 lo = __floats2bfloat162_rn(__uint_as_float(a.x) + __uint_as_float(b.x),
                                                            __uint_as_float(a.y) + __uint_as_float(b.y));
            const __nv_bfloat162 hi = __floats2bfloat162_rn(__uint_as_float(a.z) + __uint_as_float(b.z),
                                                            __uint_as_float(a.w) + __uint_as_float(b.w));
            uint2 v;
            v.x = *reinterpret_cast<const uint32_t*>(&lo);
            v.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(hs + static_cast<size_t>(t) * (p.r + 8) + k) = v;
        }
        main_sync();
    }

    // ---- Re-arm the counters for the next call on this scratch buffer.  Every CTA checks out once it is past its
    // waits, and the last one to do so (nobody reads the counters of this call any more) zeroes them.  Doing it here
    // rather than at the end keeps two atomic round trips out of the tail of the launch.
    if (threadIdx.x == 0) {
        if (atomicAdd(p.sync + 1, 1u) == static_cast<unsigned int>(G - 1)) {
            atomicExch(p.sync, 0u);
            atomicExch(p.sync + 1, 0u);
            atomicExch(p.sync + 3, 0u);
        }
    }

    // ---- phase U and store
    if (p.upf > 0) fa_cp_async_wait(0);                    // every thread reads back only its own copies
    int uk = 0;
    for (int blk = row0; blk < row1; blk += FA_ROWS) {
        float acc[2][NT][4];
        zero_acc<NT>(acc);
        uh_block<NT, SIDE>(p, acc, blk, row1, hs, ustage, uk, warp, gid, tig);
        const float* yb = ybuf + static_cast<size_t>(blk - row0) * YS;
        const int T = p.T, M = p.M;
        __nv_bfloat16* out = p.out;
        reduce_tiles<NT>(red, acc, warp, gid, tig, [=](int row, int t, float s) {
            const int m = blk + row;
            if (m < row1 && t < T) {
                const size_t o = static_cast<size_t>(t) * M + m;
                s += yb[row * YS + t];
                out[o] = __float2bfloat16_rn(s);
            }
        });
    }

}

}  // namespace ade
