// Producer side of the packed-delta format on the GPU: one pass from a factor of the truncated SVD to 4-bit codes,
// bfloat16 scales and zero-points.
//
// Replaces, for one factor X (rows x r, float32), the chain of src/quantization.py:244-285:
//     X * sqrt(S)                      (:266-268)
//     ... @ H                          (:270-272; H = normalised Sylvester Hadamard when r is a power of two, :56-70)
//     quantize_rowwise / _colwise      (:134-199, with _pin_zero_in_range :109-131)
// The reference multiplies by a dense r x r matrix (2 r^2 flops per row) and then makes about ten elementwise passes
// over the result.  Here a CTA keeps a row in shared memory, applies the Hadamard rotation as a fast Walsh-Hadamard
// transform (r log2 r additions), and quantises the row's groups of 128 where they lie: X is read once, codes, scales
// and zero-points are written once (5 bytes of traffic per element; the kernel is HBM-bound).
//
// Both factors are "rows x r" here: U is (d_o, r); V is (d_i, r), and H^T (sqrt(S) V^T) = ((V sqrt(S)) H)^T for any
// H, so the V side runs the same row kernel with its outputs written transposed (codes (r, d_i), scales and
// zero-points (r/128, d_i)), 32 rows of a CTA at a time so that the transposed writes are 32-byte segments.
//
// The quantisation arithmetic is the reference's, operation for operation in float32 (IEEE division, round half to
// even), so given the same rotated input the outputs are bit-identical to quantize_rowwise / quantize_colwise.  The
// transform sums in another order than a dense matmul, so after a rotation codes can differ by one step where a value
// sits on a rounding boundary.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ade {

constexpr int CQ_THREADS = 256;
constexpr int CQ_ROWS = 32;            // rows per CTA (one transposed write segment)
constexpr int CQ_MAX_RANK = 2048;

__host__ __device__ inline size_t compress_smem_bytes(int r, bool transposed) {
    const size_t row = static_cast<size_t>(r) * sizeof(float);
    const size_t tile = transposed ? static_cast<size_t>(r) * CQ_ROWS + static_cast<size_t>(r / 128) * CQ_ROWS * 4 : 0;
    return row + tile;
}

// X (rows, r) float32; sqrt_s (r) float32 or nullptr; rotate: in-kernel Hadamard transform (r a power of two).
// Row-wise outputs: codes (rows, r), scale / zero (rows, r/128).  Transposed: codes (r, rows), scale / zero (r/128, rows).
template <bool TRANSPOSED>
__global__ void __launch_bounds__(CQ_THREADS) compress_rows_kernel(const float* __restrict__ X, const float* __restrict__ sqrt_s,
                                                                     uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ scale,
                                                                     __nv_bfloat16* __restrict__ zero, int rows, int r, int rotate) {
    extern __shared__ float cq_smem[];
    float* row = cq_smem;                                               // [r]
    uint8_t* ctile = reinterpret_cast<uint8_t*>(row + r);               // [r][CQ_ROWS] codes (transposed only)
    __nv_bfloat16* stile = reinterpret_cast<__nv_bfloat16*>(ctile + static_cast<size_t>(r) * CQ_ROWS);   // [ng][CQ_ROWS] scale, then zero
    const int ng = r >> 7;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float norm = rotate ? rsqrtf(static_cast<float>(r)) : 1.0f;  // exact for r = 4^k, else one rounding (as 1 / sqrt(r))
    for (int m0 = blockIdx.x * CQ_ROWS; m0 < rows; m0 += gridDim.x * CQ_ROWS) {
        const int nrows = min(CQ_ROWS, rows - m0);
        for (int rr = 0; rr < nrows; ++rr) {
            const size_t m = static_cast<size_t>(m0 + rr);
            for (int k = threadIdx.x; k < r; k += CQ_THREADS) {
                const float x = X[m * r + k];
                row[k] = sqrt_s ? x * sqrt_s[k] : x;
            }
            __syncthreads();
            if (rotate) {
                for (int h = 1; h < r; h <<= 1) {
                    for (int i = threadIdx.x; i < (r >> 1); i += CQ_THREADS) {
                        const int j = ((i / h) * (h << 1)) + (i % h);
                        const float a = row[j], b = row[j + h];
                        row[j] = a + b;
                        row[j + h] = a - b;
                    }
                    __syncthreads();
                }
            }
            for (int g = warp; g < ng; g += CQ_THREADS / 32) {
                float v[4];
                float lo = 3.402823466e38f, hi = -3.402823466e38f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[i] = row[g * 128 + lane + 32 * i] * norm;
                    lo = fminf(lo, v[i]);
                    hi = fmaxf(hi, v[i]);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, o));
                    hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o));
                }
                if (lo == 0.f && hi == 0.f) {                           // an all-zero group quantises as [-1, 1]
                    lo = -1.f;
                    hi = 1.f;
                }
                float sc = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-5f), 15.f);
                float zp = rintf(__fdiv_rn(-lo, sc));
                if (zp < 0.f) {                                         // one-signed groups are widened to contain 0
                    sc = __fdiv_rn(fmaxf(hi, 1e-5f), 15.f);
                    zp = 0.f;
                } else if (zp > 15.f) {
                    sc = __fdiv_rn(fmaxf(-lo, 1e-5f), 15.f);
                    zp = 15.f;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float q = fminf(fmaxf(__fadd_rn(rintf(__fdiv_rn(v[i], sc)), zp), 0.f), 15.f);
                    const uint8_t c = static_cast<uint8_t>(q);
                    const int k = g * 128 + lane + 32 * i;
                    if (TRANSPOSED) ctile[k * CQ_ROWS + rr] = c;
                    else codes[m * r + k] = c;
                }
                if (lane == 0) {
                    if (TRANSPOSED) {
                        stile[g * CQ_ROWS + rr] = __float2bfloat16_rn(sc);
                        stile[(ng + g) * CQ_ROWS + rr] = __float2bfloat16_rn(zp);
                    } else {
                        scale[m * ng + g] = __float2bfloat16_rn(sc);
                        zero[m * ng + g] = __float2bfloat16_rn(zp);
                    }
                }
            }
            __syncthreads();
        }
        if (TRANSPOSED) {
            // codes (r, rows): row k of the output gets this CTA's nrows bytes at column m0
            for (int e = threadIdx.x; e < r * (CQ_ROWS / 4); e += CQ_THREADS) {
                const int k = e / (CQ_ROWS / 4), q4 = e % (CQ_ROWS / 4);
                uint8_t* dst = codes + static_cast<size_t>(k) * rows + m0 + 4 * q4;
                if (nrows == CQ_ROWS && (rows & 3) == 0) {
                    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(ctile + k * CQ_ROWS + 4 * q4);
                } else {
                    for (int b = 0; b < 4; ++b)
                        if (4 * q4 + b < nrows) dst[b] = ctile[k * CQ_ROWS + 4 * q4 + b];
                }
            }
            for (int e = threadIdx.x; e < ng * CQ_ROWS; e += CQ_THREADS) {
                const int g = e / CQ_ROWS, rr = e % CQ_ROWS;
                if (rr < nrows) {
                    scale[static_cast<size_t>(g) * rows + m0 + rr] = stile[g * CQ_ROWS + rr];
                    zero[static_cast<size_t>(g) * rows + m0 + rr] = stile[(ng + g) * CQ_ROWS + rr];
                }
            }
            __syncthreads();
        }
    }
}

}  // namespace ade
