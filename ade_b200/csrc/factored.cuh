// Factored application  out = base_term + U^ (V^T x)  for T <= 128 tokens.
//
// Replaces the reference's decode kernels A and B (src/kernels.py:486-886).  Two launches:
//
//   xv_kernel : h[t][k]   = sum_n bf16((Vcode[k][n] - vz[g][n]) * vs[g][n]) * x[t][n]      (fp32 accumulate)
//   hu_kernel : out[t][m] = base[t][m] + sum_g us[m][g] * sum_{k in g} (Ucode[m][k] - uz[m][g]) * h[t][k]
//               with base = y_dense (given) or  sum_n w_b[m][n] x[t][n]  streamed in the same kernel.
//
// Both are weight-streaming skinny GEMMs: the weights (bf16 rows of W_b, or 4-bit codes) are
// the 16-row operand of a warp MMA and come straight from global memory with 128-bit loads;
// the activations (x or h, a few KB that live in L1/L2) are the 8-column operand.  The
// contraction axis is split over the warps of a CTA and reduced through shared memory in a
// fixed order, so results do not depend on scheduling (no atomics).
//
// Fragment bookkeeping (mma.m16n8k16, lane = 4*gid + tig): a thread's 16-byte load covers
// 8 bf16 (or 32 codes) of one weight row; consecutive 4-element slices of it are used as the
// thread's k-slots {2tig, 2tig+1, 2tig+8, 2tig+9} of consecutive MMAs, and the activation
// fragment is read from the same 4 columns, so the products line up without any shuffle.
#pragma once
#include "ptx.cuh"

namespace ade {

constexpr int XV_WARPS = 16;
constexpr int XV_THREADS = XV_WARPS * 32;
constexpr int HU_WARPS = 8;
constexpr int HU_THREADS = HU_WARPS * 32;
constexpr int HU_ROWS = 32;          // output rows per CTA (two m16 tiles per warp)
constexpr uint32_t kBf2_128 = 0x43004300u;   // bf16x2 (128, 128)

// one packed word (8 codes) -> 4 bf16x2 registers holding 128 + code, codes in natural order
__device__ __forceinline__ void unpack8_bf16(uint32_t w, uint32_t (&e)[4]) {
    e[0] = (w & 0x000F000Fu) | kBf2_128;
    e[1] = ((w >> 4) & 0x000F000Fu) | kBf2_128;
    e[2] = ((w >> 8) & 0x000F000Fu) | kBf2_128;
    e[3] = ((w >> 12) & 0x000F000Fu) | kBf2_128;
}

// ---------------------------------------------------------------------------------------
// h = V^T x.  grid = r / 16 CTAs (16 ranks each), XV_THREADS threads; the d_i axis is split
// over the warps in chunks of 128 columns.
// ---------------------------------------------------------------------------------------
template <int NT>
__global__ void __launch_bounds__(XV_THREADS)
xv_kernel(const uint8_t* __restrict__ vt, const uint16_t* __restrict__ vs, const uint8_t* __restrict__ vz,
          const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ h, int T, int N, int r) {
    __shared__ float red[XV_WARPS][16][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int k0 = blockIdx.x * 16;
    const int g = k0 >> 7;
    const size_t rowb = static_cast<size_t>(N >> 1);
    const uint8_t* row0 = vt + static_cast<size_t>(k0 + gid) * rowb;
    const uint8_t* row1 = row0 + 8 * rowb;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

    const int nchunks = N >> 7;
    for (int c = warp; c < nchunks; c += XV_WARPS) {
        const int nb = (c << 7) + tig * 32;               // this thread's 32 columns
        const uint4 q0 = ldg16_stream(row0 + (nb >> 1));
        const uint4 q1 = ldg16_stream(row1 + (nb >> 1));
        const uint16_t* sp = vs + static_cast<size_t>(g) * N + nb;
        const uint8_t* zp = vz + static_cast<size_t>(g) * N + nb;
        const uint4 s0 = ldg16(sp), s1 = ldg16(sp + 8), s2 = ldg16(sp + 16), s3 = ldg16(sp + 24);
        const uint4 z0 = ldg16(zp), z1 = ldg16(zp + 16);
        const uint32_t cw0[4] = {q0.x, q0.y, q0.z, q0.w};
        const uint32_t cw1[4] = {q1.x, q1.y, q1.z, q1.w};
        const uint32_t sw[16] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w,
                                 s2.x, s2.y, s2.z, s2.w, s3.x, s3.y, s3.z, s3.w};
        const uint32_t zw[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
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
            for (int p = 0; p < 4; ++p) {                 // (code - zero) is exact; one rounding in the product
                a0[p] = bf2_mul(bf2_sub(e0[p], zz[p]), sw[4 * wi + p]);
                a1[p] = bf2_mul(bf2_sub(e1[p], zz[p]), sw[4 * wi + p]);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + gid;
                uint4 xq = make_uint4(0u, 0u, 0u, 0u);
                if (tok < T) xq = ldg16(x + static_cast<size_t>(tok) * N + nb + 8 * wi);
                mma_bf16(acc[nt], a0[0], a1[0], a0[1], a1[1], xq.x, xq.y);
                mma_bf16(acc[nt], a0[2], a1[2], a0[3], a1[3], xq.z, xq.w);
            }
        }
    }

    // fixed-order reduction over the warps, 32 tokens (4 token tiles) at a time
#pragma unroll
    for (int b = 0; b < (NT + 3) / 4; ++b) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nt = b * 4 + j;
            if (nt < NT) {
                red[warp][gid][j * 8 + 2 * tig] = acc[nt][0];
                red[warp][gid][j * 8 + 2 * tig + 1] = acc[nt][1];
                red[warp][gid + 8][j * 8 + 2 * tig] = acc[nt][2];
                red[warp][gid + 8][j * 8 + 2 * tig + 1] = acc[nt][3];
            }
        }
        __syncthreads();
        {
            const int rank = threadIdx.x & 15, tok = threadIdx.x >> 4;      // 16 x 32 = XV_THREADS
            const int t = b * 32 + tok;
            if (tok < 8 * (NT - 4 * b) && t < T) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < XV_WARPS; ++w) s += red[w][rank][tok];
                h[static_cast<size_t>(t) * r + k0 + rank] = __float2bfloat16_rn(s);
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// out = base + U^ h.  grid = M / 32 CTAs, HU_THREADS threads.
// ---------------------------------------------------------------------------------------
template <int NT, bool FUSE_WB>
__global__ void __launch_bounds__(HU_THREADS)
hu_kernel(const __nv_bfloat16* __restrict__ w_b, const __nv_bfloat16* __restrict__ x,
          const __nv_bfloat16* __restrict__ y_dense, const uint8_t* __restrict__ uq,
          const uint16_t* __restrict__ us, const uint8_t* __restrict__ uz,
          const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out, int T, int M, int N, int r) {
    __shared__ float red[HU_WARPS][32][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int m0 = blockIdx.x * HU_ROWS;

    float acc[2][NT][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

    if (FUSE_WB) {
        // W_b x: contraction over d_i in blocks of 64 columns, block b -> warp b % HU_WARPS
        const int nblk = N >> 6;
        const __nv_bfloat16* wrow[2][2];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            wrow[mt][0] = w_b + static_cast<size_t>(m0 + mt * 16 + gid) * N + tig * 8;
            wrow[mt][1] = wrow[mt][0] + static_cast<size_t>(8) * N;
        }
        uint4 cur[2][2][2], nxt[2][2][2];
        if (warp < nblk) {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr)
#pragma unroll
                    for (int s = 0; s < 2; ++s) cur[mt][hr][s] = ldg16_stream(wrow[mt][hr] + warp * 64 + s * 32);
        }
        for (int b = warp; b < nblk; b += HU_WARPS) {
            const int bn = b + HU_WARPS;
            if (bn < nblk) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int hr = 0; hr < 2; ++hr)
#pragma unroll
                        for (int s = 0; s < 2; ++s) nxt[mt][hr][s] = ldg16_stream(wrow[mt][hr] + bn * 64 + s * 32);
            }
            const int kb = b * 64 + tig * 8;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + gid;
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    uint4 xq = make_uint4(0u, 0u, 0u, 0u);
                    if (tok < T) xq = ldg16(x + static_cast<size_t>(tok) * N + kb + s * 32);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        mma_bf16(acc[mt][nt], cur[mt][0][s].x, cur[mt][1][s].x, cur[mt][0][s].y, cur[mt][1][s].y,
                                 xq.x, xq.y);
                        mma_bf16(acc[mt][nt], cur[mt][0][s].z, cur[mt][1][s].z, cur[mt][0][s].w, cur[mt][1][s].w,
                                 xq.z, xq.w);
                    }
                }
            }
            if (bn < nblk) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int hr = 0; hr < 2; ++hr)
#pragma unroll
                        for (int s = 0; s < 2; ++s) cur[mt][hr][s] = nxt[mt][hr][s];
            }
        }
    }

    // U^ h: one rank group (128 ranks) per warp iteration, group g -> warp g % HU_WARPS
    {
        const int ng = r >> 7;
        const size_t rowb = static_cast<size_t>(r >> 1);
        for (int g = warp; g < ng; g += HU_WARPS) {
            uint32_t a[2][2][16];        // [m16 tile][row gid / gid+8][pair]: (code - zero) as bf16x2
            float su[2][2];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    const int m = m0 + mt * 16 + hr * 8 + gid;
                    const uint4 q = ldg16_stream(uq + static_cast<size_t>(m) * rowb + g * 64 + tig * 16);
                    const uint32_t z = uz[static_cast<size_t>(m) * ng + g];
                    const uint32_t zz = kBf2_128 | z | (z << 16);
                    su[mt][hr] = bf16_bits_to_f32(us[static_cast<size_t>(m) * ng + g]);
                    const uint32_t cw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) {
                        uint32_t e[4];
                        unpack8_bf16(cw[wi], e);
#pragma unroll
                        for (int p = 0; p < 4; ++p) a[mt][hr][4 * wi + p] = bf2_sub(e[p], zz);
                    }
                }
            const int kb = g * 128 + tig * 32;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + gid;
                float pa[2][4];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) pa[mt][i] = 0.f;
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    uint4 hq = make_uint4(0u, 0u, 0u, 0u);
                    if (tok < T) hq = ldg16(h + static_cast<size_t>(tok) * r + kb + 8 * wi);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        mma_bf16(pa[mt], a[mt][0][4 * wi], a[mt][1][4 * wi], a[mt][0][4 * wi + 1], a[mt][1][4 * wi + 1],
                                 hq.x, hq.y);
                        mma_bf16(pa[mt], a[mt][0][4 * wi + 2], a[mt][1][4 * wi + 2], a[mt][0][4 * wi + 3],
                                 a[mt][1][4 * wi + 3], hq.z, hq.w);
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {          // one rescale per group
                    acc[mt][nt][0] += su[mt][0] * pa[mt][0];
                    acc[mt][nt][1] += su[mt][0] * pa[mt][1];
                    acc[mt][nt][2] += su[mt][1] * pa[mt][2];
                    acc[mt][nt][3] += su[mt][1] * pa[mt][3];
                }
            }
        }
    }

    // fixed-order reduction over the warps and store, 32 tokens at a time
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
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * HU_THREADS;
            const int row = e & 31, tok = e >> 5;
            const int t = b * 32 + tok;
            if (tok < 8 * (NT - 4 * b) && t < T) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < HU_WARPS; ++w) s += red[w][tok][row];
                const size_t o = static_cast<size_t>(t) * M + m0 + row;
                if (!FUSE_WB) s += __bfloat162float(y_dense[o]);
                out[o] = __float2bfloat16_rn(s);
            }
        }
        __syncthreads();
    }
}

}  // namespace ade
