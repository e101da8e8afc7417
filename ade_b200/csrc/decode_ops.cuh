// Small fused kernels for the token-by-token decode step of a LLaMA-architecture model.
//
// They are not part of the delta application itself.  At decode sizes a Hugging Face decoder layer runs about forty
// elementwise kernels around the four launches of the factored kernel (RMSNorm: 8 each, rotary embedding: 14, SiLU
// and product: 2), and inside a CUDA graph every one of them costs about as much as it would take to stream a
// megabyte of weights.  The three kernels here do the same arithmetic with the same bfloat16 roundings in one launch
// each, so that tokens/s measures the weight stream and not the launch count; a fourth does the single-token attention
// step (rotary embedding, KV-cache write, attention) in one launch.  No counterpart in the reference, which leaves
// these operations to transformers (src/evaluate.py:241 calls model.generate).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ade {

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// out[t][:] = w * bf16(x[t][:] * rsqrt(mean(x[t][:]^2) + eps)): float32 statistics, the normalised value rounded to
// bfloat16 before the (bfloat16) multiplication by the weight, as LlamaRMSNorm.forward does.  One CTA per row.
// With `res` the row normalised is s = bf16(x + res) (the residual connection, rounded as torch rounds the sum of two
// bfloat16 tensors) and s is written to `sum_out` as well: residual add and the following RMSNorm in one launch.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ sum_out,
                                                       __nv_bfloat16* __restrict__ out, int H, long long x_stride, long long res_stride,
                                                       float eps) {
    __shared__ float part[8];
    const __nv_bfloat16* xr = x + static_cast<size_t>(blockIdx.x) * x_stride;
    const __nv_bfloat16* rr = res ? res + static_cast<size_t>(blockIdx.x) * res_stride : nullptr;
    __nv_bfloat16* srow = sum_out ? sum_out + static_cast<size_t>(blockIdx.x) * H : nullptr;
    __nv_bfloat16* orow = out + static_cast<size_t>(blockIdx.x) * H;
    // 16-byte pieces (8 values), up to four per thread kept in registers between the two passes (rows up to 8192 wide);
    // rows that are wider, not a multiple of 8 or not 16-byte aligned take the element-wise loops
    const bool vec = (H & 7) == 0 && H <= 8192 &&
                     ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(rr)) & 15) == 0;
    const int nvec = H >> 3;
    uint4 xv[4], wv4[4];
    float s = 0.f;
    if (vec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x + k * 256;
            xv[k] = make_uint4(0u, 0u, 0u, 0u);
            wv4[k] = make_uint4(0u, 0u, 0u, 0u);
            if (i < nvec) {
                wv4[k] = reinterpret_cast<const uint4*>(w)[i];       // requested together with the row: one memory round trip
                xv[k] = reinterpret_cast<const uint4*>(xr)[i];
                if (rr) {
                    const uint4 rv = reinterpret_cast<const uint4*>(rr)[i];
                    uint32_t xx[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
                    const uint32_t r4[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(xx[e] << 16) + __uint_as_float(r4[e] << 16),
                                                                        __uint_as_float(xx[e] & 0xFFFF0000u) + __uint_as_float(r4[e] & 0xFFFF0000u));
                        xx[e] = *reinterpret_cast<const uint32_t*>(&o);
                    }
                    xv[k] = make_uint4(xx[0], xx[1], xx[2], xx[3]);
                    reinterpret_cast<uint4*>(srow)[i] = xv[k];
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t ww[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float a = __uint_as_float(ww[e] << 16), c = __uint_as_float(ww[e] & 0xFFFF0000u);
                s += a * a;
                s += c * c;
            }
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = __bfloat162float(xr[i]);
            if (rr) {
                v = bf16r(v + __bfloat162float(rr[i]));
                srow[i] = __float2bfloat16_rn(v);
            }
            s += v * v;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
    if (vec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < nvec) {
                const uint32_t xx[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
                const uint32_t ww[4] = {wv4[k].x, wv4[k].y, wv4[k].z, wv4[k].w};
                uint32_t oo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float n0 = bf16r(__uint_as_float(xx[e] << 16) * inv), n1 = bf16r(__uint_as_float(xx[e] & 0xFFFF0000u) * inv);
                    const __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(ww[e] << 16) * n0, __uint_as_float(ww[e] & 0xFFFF0000u) * n1);
                    oo[e] = *reinterpret_cast<const uint32_t*>(&o);
                }
                reinterpret_cast<uint4*>(orow)[i] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
            }
        }
    } else {
        const __nv_bfloat16* src = rr ? srow : xr;           // the sum was written above by this very thread
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float n = bf16r(__bfloat162float(src[i]) * inv);
            orow[i] = __float2bfloat16_rn(__bfloat162float(w[i]) * n);
        }
    }
}

// Rotary position embedding of q and k in one launch (apply_rotary_pos_emb of transformers' LLaMA model):
//   out[i] = bf16(bf16(x[i] cos[i]) + bf16(rot[i] sin[i])),  rot = (-x[hd/2:], x[:hd/2]),
// every product and the sum rounded to bfloat16 as the elementwise torch operations round them.
// x is read as [B][T][heads][hd] with a row stride (the projections may be column slices of a fused output); the
// result is written as [B][heads][T][hd], the layout attention and the KV cache take.  cos / sin: [B or 1][T][hd]
// (cs_batch_stride = T * hd, or 0 when one table serves every batch row).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ cs,
                            const __nv_bfloat16* __restrict__ sn, __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko, int B, int T,
                            int hq, int hk, int hd, long long q_stride, long long k_stride, long long cs_batch_stride) {
    const int half = hd >> 1;
    const long long total = static_cast<long long>(B) * T * (hq + hk) * hd;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total; e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(e % hd);
        long long r = e / hd;
        const int h = static_cast<int>(r % (hq + hk));
        r /= (hq + hk);
        const int t = static_cast<int>(r % T), b = static_cast<int>(r / T);
        const bool is_q = h < hq;
        const int hh = is_q ? h : h - hq;
        const __nv_bfloat16* src = (is_q ? q + (static_cast<long long>(b) * T + t) * q_stride : k + (static_cast<long long>(b) * T + t) * k_stride) + hh * hd;
        const float x = __bfloat162float(src[d]);
        const float other = d < half ? -__bfloat162float(src[d + half]) : __bfloat162float(src[d - half]);
        const size_t ci = static_cast<size_t>(b) * cs_batch_stride + static_cast<size_t>(t) * hd + d;
        const float v = bf16r(bf16r(x * __bfloat162float(cs[ci])) + bf16r(other * __bfloat162float(sn[ci])));
        __nv_bfloat16* dst = is_q ? qo + ((static_cast<size_t>(b) * hq + hh) * T + t) * hd : ko + ((static_cast<size_t>(b) * hk + hh) * T + t) * hd;
        dst[d] = __float2bfloat16_rn(v);
    }
}

// out = bf16(bf16(silu(g)) * u), silu evaluated in float32 as torch evaluates it for a bfloat16 tensor.
// g and u are [rows][cols] with row strides (column slices of a fused gate/up output), out is contiguous.
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ out,
                                int rows, int cols, long long g_stride, long long u_stride) {
    const long long total = static_cast<long long>(rows) * cols;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total; e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = e / cols;
        const int c = static_cast<int>(e - r * cols);
        const float x = __bfloat162float(g[r * g_stride + c]);
        const float s = bf16r(x / (1.0f + expf(-x)));
        out[e] = __float2bfloat16_rn(s * __bfloat162float(u[r * u_stride + c]));
    }
}

// One decode step of attention for one new token per sequence: rotary embedding of q and k, the write of k and v into
// the static KV cache at position *pos, and softmax(q K^T * scale) V over the cache positions the mask allows, in one
// launch (transformers runs the rotary embedding, two index_copy_ calls with their index arithmetic and scaled dot
// product attention as about twenty kernels here).  One CTA of 128 threads per (sequence, query head).
//   q [B][hq*hd], k / v [B][hk*hd] with row strides (column slices of a fused q/k/v output); cos / sin [B or 1][hd];
//   kc / vc: the cache, [B][hk][L][hd] contiguous; mask: bool [B][L], true = attend (it includes position *pos), or
//   nullptr = attend to positions 0 .. *pos; out [B][hq*hd] contiguous.
// The new k (rotated, rounded to bfloat16 as the cache stores it) and v are used from registers for position *pos, so
// no CTA reads what another one writes in the same launch; the CTA of the first query head of every KV group writes
// them to the cache.  Scores, softmax and the weighted sum are float32.  With `ticket` (a zero-initialised counter of
// its own per cache layer) the launch also advances *pos by one once every CTA has read it.
__global__ void __launch_bounds__(128) attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                           const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ cs,
                                                           const __nv_bfloat16* __restrict__ sn, const bool* __restrict__ mask,
                                                           __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                                           long long* __restrict__ pos, unsigned int* __restrict__ ticket,
                                                           __nv_bfloat16* __restrict__ out, int hq, int hk,
                                                           int hd, int L, long long q_stride, long long k_stride, long long v_stride,
                                                           long long cs_batch_stride, long long mask_stride, float scale) {
    extern __shared__ float at_smem[];
    float* qs = at_smem;              // [hd] rotated q
    float* kn = qs + hd;              // [hd] rotated new k (bfloat16 values)
    float* vn = kn + hd;              // [hd] new v
    float* red = vn + hd;             // [4 warps][hd] partial sums / [128] reductions
    float* sc = red + 4 * hd;         // [L] scores, then weights
    const int b = blockIdx.x / hq, h = blockIdx.x % hq;
    const int group = hq / hk, kvh = h / group;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p0 = static_cast<int>(*pos);
    if (ticket != nullptr) {
        // every CTA has read the position by the time the last ticket is drawn: that CTA advances it for the next
        // step and re-arms the counter (nobody reads *pos again in this launch)
        __syncthreads();
        if (tid == 0 && atomicAdd(ticket, 1u) == gridDim.x - 1) {
            *pos = p0 + 1;
            *ticket = 0u;
        }
    }
    const int half = hd >> 1;
    const __nv_bfloat16* qr = q + static_cast<size_t>(b) * q_stride + h * hd;
    const __nv_bfloat16* kr = k + static_cast<size_t>(b) * k_stride + kvh * hd;
    const __nv_bfloat16* vr = v + static_cast<size_t>(b) * v_stride + kvh * hd;
    __nv_bfloat16* kcb = kc + (static_cast<size_t>(b) * hk + kvh) * L * hd;
    __nv_bfloat16* vcb = vc + (static_cast<size_t>(b) * hk + kvh) * L * hd;
    for (int d = tid; d < hd; d += 128) {
        const float c = __bfloat162float(cs[static_cast<size_t>(b) * cs_batch_stride + d]);
        const float s = __bfloat162float(sn[static_cast<size_t>(b) * cs_batch_stride + d]);
        const int od = d < half ? d + half : d - half;
        const float sign = d < half ? -1.f : 1.f;
        qs[d] = bf16r(bf16r(__bfloat162float(qr[d]) * c) + bf16r(sign * __bfloat162float(qr[od]) * s));
        kn[d] = bf16r(bf16r(__bfloat162float(kr[d]) * c) + bf16r(sign * __bfloat162float(kr[od]) * s));
        vn[d] = __bfloat162float(vr[d]);
        if (h % group == 0 && p0 >= 0 && p0 < L) {
            kcb[static_cast<size_t>(p0) * hd + d] = __float2bfloat16_rn(kn[d]);
            vcb[static_cast<size_t>(p0) * hd + d] = vr[d];
        }
    }
    __syncthreads();
    // scores: one cache position per thread and pass
    const bool* mb = mask ? mask + static_cast<size_t>(b) * mask_stride : nullptr;
    float mx = -3.0e38f;
    int hi = 0;                                            // one past the last attended position
    for (int p = tid; p < L; p += 128) {
        const bool on = mb ? mb[p] : p <= p0;
        float s = -3.0e38f;
        if (on) {
            float a = 0.f;
            if (p == p0) {
                for (int d = 0; d < hd; ++d) a += qs[d] * kn[d];
            } else {
                const uint4* row = reinterpret_cast<const uint4*>(kcb + static_cast<size_t>(p) * hd);
#pragma unroll 8
                for (int c8 = 0; c8 < (hd >> 3); ++c8) {
                    const uint4 w = row[c8];
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        a += qs[c8 * 8 + 2 * e] * __uint_as_float(ww[e] << 16);
                        a += qs[c8 * 8 + 2 * e + 1] * __uint_as_float(ww[e] & 0xFFFF0000u);
                    }
                }
            }
            s = a * scale;
            hi = p + 1;
        }
        sc[p] = s;
        mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        hi = max(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o));
    }
    if (lane == 0) {
        red[warp] = mx;
        red[4 + warp] = static_cast<float>(hi);
    }
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    hi = static_cast<int>(fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
    __syncthreads();
    float sum = 0.f;
    for (int p = tid; p < hi; p += 128) {
        const float w = sc[p] > -1.0e38f ? expf(sc[p] - mx) : 0.f;
        sc[p] = w;
        sum += w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = red[0] + red[1] + red[2] + red[3];
    __syncthreads();
    // weighted sum of v: a thread owns 8 consecutive dimensions (one 16-byte piece of a cache row) and every
    // (128 / (hd / 8))-th position, up to sixteen rows in flight at a time; the position lanes are summed through shared
    // memory
    const int chunks = hd >> 3;                            // 16-byte pieces per row: 4 .. 32
    const int lanes_p = 128 / chunks;                      // position lanes: 32 .. 4
    const int c8 = tid % chunks, pl = tid / chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add_row = [&](const uint4& w, float wt) {
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc[2 * e] += wt * __uint_as_float(ww[e] << 16);
            acc[2 * e + 1] += wt * __uint_as_float(ww[e] & 0xFFFF0000u);
        }
    };
    if (pl < lanes_p) {
        const uint4* vrow = reinterpret_cast<const uint4*>(vcb) + c8;
        const int stride = chunks;                         // uint4 per row
        int p = pl;
        for (; p + 15 * lanes_p < hi; p += 16 * lanes_p) {     // long caches: sixteen rows in flight
            uint4 w4[16];
            float wt[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int pp = p + u * lanes_p;
                wt[u] = pp == p0 ? 0.f : sc[pp];
                w4[u] = vrow[static_cast<size_t>(pp) * stride];
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) add_row(w4[u], wt[u]);
        }
        for (; p + 7 * lanes_p < hi; p += 8 * lanes_p) {
            uint4 w4[8];
            float wt[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int pp = p + u * lanes_p;
                wt[u] = pp == p0 ? 0.f : sc[pp];
                w4[u] = vrow[static_cast<size_t>(pp) * stride];
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) add_row(w4[u], wt[u]);
        }
        for (; p + 3 * lanes_p < hi; p += 4 * lanes_p) {
            uint4 w4[4];
            float wt[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int pp = p + u * lanes_p;
                wt[u] = pp == p0 ? 0.f : sc[pp];           // the new token's row is added from registers below
                w4[u] = vrow[static_cast<size_t>(pp) * stride];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) add_row(w4[u], wt[u]);
        }
        for (; p < hi; p += lanes_p)
            if (p != p0) add_row(vrow[static_cast<size_t>(p) * stride], sc[p]);
        if (pl == 0 && p0 >= 0 && p0 < hi) {
            const float wt = sc[p0];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += wt * vn[c8 * 8 + i];
        }
    }
    __syncthreads();                                       // sc is no longer read: reuse it with red for the lane sums
    // the position lanes are folded into lane 0 four at a time through red ([4][hd] floats)
    for (int round = 0; round < lanes_p; round += 4) {
        if (pl >= round && pl < round + 4 && pl < lanes_p)
            for (int i = 0; i < 8; ++i) red[(pl - round) * hd + c8 * 8 + i] = acc[i];
        __syncthreads();
        if (pl == 0) {
            const int n = min(4, lanes_p - round);
            for (int i = 0; i < 8; ++i) {
                float t = 0.f;
                for (int j = (round == 0 ? 1 : 0); j < n; ++j) t += red[j * hd + c8 * 8 + i];
                acc[i] += t;
            }
        }
        __syncthreads();
    }
    if (pl == 0) {
        __nv_bfloat16* o = out + (static_cast<size_t>(b) * hq + h) * hd + c8 * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(acc[i] / sum);
    }
}

// The same step as attn_decode_kernel for head dimensions 32, 64, 128 and 256, as ONE pass over the cache with a running
// softmax: CH = hd / 8 lanes share a cache row (a lane owns 8 consecutive dimensions, one 16-byte piece of the k row and
// of the v row), so a warp's load instruction covers 32 / CH whole rows and the 128 / CH row groups of the CTA read
// consecutive rows; twelve k rows and twelve v rows are in flight per thread.  The partial products of a row are added
// over its lanes with shuffles; every group keeps (running maximum, running sum, weighted sum of v) and the groups are
// combined through shared memory at the end.  attn_decode_kernel reads k one position per thread (32 different rows
// per load instruction) and walks the cache twice.
template <int CH>
__global__ void __launch_bounds__(128) attn_decode_stream_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                                  const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ cs,
                                                                  const __nv_bfloat16* __restrict__ sn, const bool* __restrict__ mask,
                                                                  __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                                                  long long* __restrict__ pos, unsigned int* __restrict__ ticket,
                                                                  __nv_bfloat16* __restrict__ out, int hq, int hk, int L, long long q_stride,
                                                                  long long k_stride, long long v_stride, long long cs_batch_stride,
                                                                  long long mask_stride, float scale) {
    constexpr int hd = CH * 8, G = 128 / CH, U = 12;       // rows in flight per thread (8: 25.8 us, 12: 20.5, 16: 22.2 at batch 8 with 540 cached positions)
    __shared__ float qs[hd], kn[hd], vn[hd];
    __shared__ float st[G][hd + 2];                        // per row group: maximum, sum, weighted sum of v
    const int b = blockIdx.x / hq, h = blockIdx.x % hq;
    const int group = hq / hk, kvh = h / group;
    const int tid = threadIdx.x;
    const int p0 = static_cast<int>(*pos);
    if (ticket != nullptr) {
        __syncthreads();
        if (tid == 0 && atomicAdd(ticket, 1u) == gridDim.x - 1) {      // see attn_decode_kernel
            *pos = p0 + 1;
            *ticket = 0u;
        }
    }
    constexpr int half = hd >> 1;
    const __nv_bfloat16* qr = q + static_cast<size_t>(b) * q_stride + h * hd;
    const __nv_bfloat16* kr = k + static_cast<size_t>(b) * k_stride + kvh * hd;
    const __nv_bfloat16* vr = v + static_cast<size_t>(b) * v_stride + kvh * hd;
    __nv_bfloat16* kcb = kc + (static_cast<size_t>(b) * hk + kvh) * L * hd;
    __nv_bfloat16* vcb = vc + (static_cast<size_t>(b) * hk + kvh) * L * hd;
    const int c8 = tid % CH, grp = tid / CH;
    const bool* mb = mask ? mask + static_cast<size_t>(b) * mask_stride : nullptr;
    const int pend = mb ? L : min(p0 + 1, L);              // positions to look at (without a mask: 0 .. *pos)
    const uint4* krow = reinterpret_cast<const uint4*>(kcb) + c8;
    const uint4* vrow = reinterpret_cast<const uint4*>(vcb) + c8;
    // Rows base + u G + grp, u = 0 .. U - 1, form a batch.  The k rows of the next batch are requested as soon as the
    // scores of the current one have been formed (their registers are free then) and its v rows once the current ones
    // have been accumulated, so loads are in flight under both halves of the arithmetic.
    uint4 kq[U], vq[U];
    uint32_t onm = 0;                                       // bit u: row u of the batch is attended to and comes from the cache
    auto rows_on = [&](int base) {
        uint32_t mk = 0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int pp = base + u * G + grp;
            if (pp < pend && pp != p0 && (mb ? mb[pp] : true)) mk |= 1u << u;      // the new token's row comes from registers below
        }
        return mk;
    };
    auto load_rows = [&](uint4 (&dst)[U], const uint4* rows, int base, uint32_t mk) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            dst[u] = make_uint4(0u, 0u, 0u, 0u);
            if (mk >> u & 1u) dst[u] = rows[static_cast<size_t>(base + u * G + grp) * CH];
        }
    };
    if (pend > 0) {                                         // the first batch travels while q and k are being rotated
        onm = rows_on(0);
        load_rows(kq, krow, 0, onm);
        load_rows(vq, vrow, 0, onm);
    }
    for (int d = tid; d < hd; d += 128) {
        const float c = __bfloat162float(cs[static_cast<size_t>(b) * cs_batch_stride + d]);
        const float s = __bfloat162float(sn[static_cast<size_t>(b) * cs_batch_stride + d]);
        const int od = d < half ? d + half : d - half;
        const float sign = d < half ? -1.f : 1.f;
        qs[d] = bf16r(bf16r(__bfloat162float(qr[d]) * c) + bf16r(sign * __bfloat162float(qr[od]) * s));
        kn[d] = bf16r(bf16r(__bfloat162float(kr[d]) * c) + bf16r(sign * __bfloat162float(kr[od]) * s));
        vn[d] = __bfloat162float(vr[d]);
        if (h % group == 0 && p0 >= 0 && p0 < L) {
            kcb[static_cast<size_t>(p0) * hd + d] = __float2bfloat16_rn(kn[d]);
            vcb[static_cast<size_t>(p0) * hd + d] = vr[d];
        }
    }
    __syncthreads();
    float qv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qv[i] = qs[c8 * 8 + i];
    float m = -3.0e38f, l = 0.f;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto dot8 = [&](const uint4& w) {
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            a += qv[2 * e] * __uint_as_float(ww[e] << 16);
            a += qv[2 * e + 1] * __uint_as_float(ww[e] & 0xFFFF0000u);
        }
        return a;
    };
    for (int base = 0; base < pend; base += U * G) {
        float sv[U];
        float bm = -3.0e38f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float a = dot8(kq[u]);
#pragma unroll
            for (int o = CH >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
            sv[u] = (onm >> u & 1u) ? a * scale : -3.0e38f;
            bm = fmaxf(bm, sv[u]);
        }
        const int nbase = base + U * G;
        const uint32_t onn = nbase < pend ? rows_on(nbase) : 0u;
        if (nbase < pend) load_rows(kq, krow, nbase, onn);
        if (bm > -1.0e38f) {                                // uniform over the group's lanes
            const float mn = fmaxf(m, bm);
            const float f = expf(m - mn);                   // 0 for the first rows of the group
            l *= f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= f;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float w = (onm >> u & 1u) ? expf(sv[u] - mn) : 0.f;
                l += w;
                const uint32_t ww[4] = {vq[u].x, vq[u].y, vq[u].z, vq[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[2 * e] += w * __uint_as_float(ww[e] << 16);
                    acc[2 * e + 1] += w * __uint_as_float(ww[e] & 0xFFFF0000u);
                }
            }
            m = mn;
        }
        if (nbase < pend) load_rows(vq, vrow, nbase, onn);
        onm = onn;
    }
    // the new token itself (its k and v have not been read back from the cache): row group 0
    {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) a += qv[i] * kn[c8 * 8 + i];
#pragma unroll
        for (int o = CH >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
        if (grp == 0 && p0 >= 0 && p0 < L && (mb ? mb[p0] : true)) {
            const float s0 = a * scale, mn = fmaxf(m, s0), f = expf(m - mn), w = expf(s0 - mn);
            l = l * f + w;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = acc[i] * f + w * vn[c8 * 8 + i];
            m = mn;
        }
    }
    if (c8 == 0) {
        st[grp][0] = m;
        st[grp][1] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) st[grp][2 + c8 * 8 + i] = acc[i];
    __syncthreads();
    if (tid < CH) {                                         // c8 == tid: 8 output dimensions per thread
        float M = -3.0e38f;
        for (int g = 0; g < G; ++g) M = fmaxf(M, st[g][0]);
        float den = 0.f, num[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int g = 0; g < G; ++g) {
            const float f = st[g][0] > -1.0e38f ? expf(st[g][0] - M) : 0.f;     // a group that attended to nothing
            den += f * st[g][1];
#pragma unroll
            for (int i = 0; i < 8; ++i) num[i] += f * st[g][2 + tid * 8 + i];
        }
        __nv_bfloat16* o = out + (static_cast<size_t>(b) * hq + h) * hd + tid * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(num[i] / den);
    }
}

}  // namespace ade
