// Reconstructed application  W' = W_b + sum_g (us (x) vs) * P_g,  P_g = <Ucode - uz, Vcode - vz> over
// the 128 ranks of group g, contracted exactly in INT32 on the 5th-generation tensor cores.
//
// Replaces ade_recon_int4_kernel (src/kernels.py:262-381); arithmetic and rounding order are
// those of the reference's PyTorch statement of eq. (7) (src/quantization.py:303-315) followed
// by the base add of src/serving.py:92.
//
// One persistent CTA per SM walks 128 x 128 output tiles.  Warp roles:
//   warps 0-7   epilogue: tcgen05.ld of P_g, float conversion, per-group rescale in FP32
//               registers (64 accumulators per thread), base add, bf16 store.  Warp w owns
//               tensor-memory lanes 32*(w%4).. and columns 64*(w/4)..
//   warps 8-11  unpack: 128-bit loads of the nibble-packed codes, expand to signed int8 with
//               the zero-point subtracted, write K-major 128-byte-swizzled operand tiles.
//   warp  12    one thread issues 4 x tcgen05.mma.kind::i8 (M=128, N=128, K=32) per group and
//               commits to mbarriers; it also owns the tensor-memory allocation.
// Rings: 3 operand stages in shared memory (32 KB each), 2 accumulator stages in tensor
// memory (128 columns each).  Every mbarrier wait is bounded: when it expires the kernel
// raises a shared abort flag, records a code in *status, lets every later wait fall through
// and still runs to its normal end (tensor memory is released, no trap).
#pragma once
#include "ptx.cuh"

namespace ade {

constexpr int RC_TILE = 128;
constexpr int RC_STAGES = 3;
constexpr int RC_STAGE_BYTES = 2 * RC_TILE * 128;      // A tile + B tile, 128 int8 per row
constexpr int RC_EPI_THREADS = 256;
constexpr int RC_PROD_THREADS = 128;
constexpr int RC_THREADS = RC_EPI_THREADS + RC_PROD_THREADS + 32;
constexpr int RC_TMEM_COLS = 256;
constexpr long long RC_SPIN_LIMIT = 2000000000LL;       // clock cycles (about one second)
// instruction descriptor: D = S32 (bits 4-5 = 2), A = B = signed 8-bit (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 = 16 (bits 17-22), M >> 4 = 8 (bits 24-28)
constexpr uint32_t RC_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | (16u << 17) | (8u << 24);

struct ReconParams {
    const uint8_t* uq;
    const uint8_t* vq;
    const uint16_t* us;
    const uint8_t* uz;
    const uint16_t* vs;
    const uint8_t* vz;
    const __nv_bfloat16* wb;
    __nv_bfloat16* out;
    int32_t* dbg;
    int* status;
    int M, N, r;
};

constexpr int RC_WB_SLOT = 144;                         // 128 bytes of W_b per epilogue thread, padded (bank spread)
constexpr int RC_WB_BYTES = RC_EPI_THREADS * RC_WB_SLOT;

__host__ __device__ inline size_t recon_smem_bytes(int ng) {
    return 1024 /* alignment slack */ + static_cast<size_t>(RC_STAGES) * RC_STAGE_BYTES + RC_WB_BYTES +
           static_cast<size_t>(4) * ng * RC_TILE * sizeof(float) + 256;
}

__device__ __forceinline__ void wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                             int code) {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return;
        if (clock64() - t0 > RC_SPIN_LIMIT) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, code);
            return;
        }
    }
}

// 32 packed codes (one 16-byte load) of operand row `row`, 16-byte column c of the packed row:
// expand to 32 signed bytes (code - zero) and store them as logical 16-byte chunks 2c, 2c+1 of
// the 128-byte row, XOR-swizzled with the row index as the 128-byte swizzle mode expects.
__device__ __forceinline__ void unpack_store(uint8_t* tile, int row, int c, uint4 q, uint32_t z) {
    const uint32_t zk = 0x80808080u - z * 0x01010101u;   // per byte 0x80 - zero, no borrow (zero <= 15)
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = w[i] & 0x0F0F0F0Fu;
        const uint32_t hi = (w[i] >> 4) & 0x0F0F0F0Fu;
        o[2 * i] = (lo + zk) ^ 0x80808080u;               // per byte code - zero, two's complement
        o[2 * i + 1] = (hi + zk) ^ 0x80808080u;
    }
    uint8_t* rp = tile + row * 128;
    const int sw = row & 7;
    *reinterpret_cast<uint4*>(rp + (((2 * c) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(rp + (((2 * c + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
}

struct ProdRegs {
    uint4 qa[4], qb[4];
    uint32_t za[4], zb[4];
};

__device__ __forceinline__ void prod_load(ProdRegs& R, const ReconParams& p, int ng, int m0, int n0, int g, int rbase,
                                          int c) {
    const size_t rowb = static_cast<size_t>(p.r >> 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = rbase + 32 * i;
        const int m = m0 + row, n = n0 + row;
        if (m < p.M) {
            R.qa[i] = ldg16(p.uq + static_cast<size_t>(m) * rowb + g * 64 + c * 16);
            R.za[i] = p.uz[static_cast<size_t>(m) * ng + g];
        } else {
            R.qa[i] = make_uint4(0u, 0u, 0u, 0u);
            R.za[i] = 0u;
        }
        R.qb[i] = ldg16(p.vq + static_cast<size_t>(n) * rowb + g * 64 + c * 16);
        R.zb[i] = p.vz[static_cast<size_t>(g) * p.N + n];
    }
}

// DBG = true additionally dumps every P_g to p.dbg (test builds of the launch only).
template <bool DBG>
__global__ void __launch_bounds__(RC_THREADS, 1) recon_kernel(const ReconParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int ng = p.r >> 7;
    uint8_t* stage_base = smem;
    uint8_t* wb_stage = smem + RC_STAGES * RC_STAGE_BYTES;                            // [256][144]
    float* sc = reinterpret_cast<float*>(wb_stage + RC_WB_BYTES);                     // [2][u|v][ng][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 4 * ng * RC_TILE);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8 * RC_STAGES;
    const uint32_t tfull0 = empty0 + 8 * RC_STAGES;
    const uint32_t tempty0 = tfull0 + 16;
    const uint32_t wbfull = tempty0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * RC_STAGES + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RC_STAGES; ++s) {
            mbar_init(full0 + 8 * s, RC_PROD_THREADS);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull0 + 8 * a, 1);
            mbar_init(tempty0 + 8 * a, RC_EPI_THREADS);
        }
        mbar_init(wbfull, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 12) {
        tmem_alloc(smem_u32(tmem_slot), RC_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_n = p.N >> 7;
    const int ntiles = ((p.M + RC_TILE - 1) >> 7) * tiles_n;

    if (warp < 8) {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3, hh = warp >> 2;
        const int row = q * 32 + lane;
        const int et = threadIdx.x;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hh * 64;
        uint32_t it = 0, tcount = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
            const int m0 = (tile / tiles_n) << 7, n0 = (tile % tiles_n) << 7;
            const int m = m0 + row;
            const bool live = m < p.M;
            float* su = sc + (tcount & 1) * (2 * ng * RC_TILE);
            float* sv = su + ng * RC_TILE;
            for (int e = et; e < ng * RC_TILE; e += RC_EPI_THREADS) {
                const int g = e >> 7, i = e & 127;
                const int mm = m0 + i;
                su[e] = mm < p.M ? bf16_bits_to_f32(p.us[static_cast<size_t>(mm) * ng + g]) : 0.f;
                sv[e] = bf16_bits_to_f32(p.vs[static_cast<size_t>(g) * p.N + n0 + i]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(RC_EPI_THREADS) : "memory");

            // this thread's 128 bytes of the base row, copied asynchronously into its own slot
            const size_t obase = static_cast<size_t>(m) * p.N + n0 + hh * 64;
            uint8_t* slot = wb_stage + et * RC_WB_SLOT;
            if (et == 0) {
                const int live_rows = min(RC_TILE, p.M - m0);
                mbar_arrive_expect_tx(wbfull, static_cast<uint32_t>(live_rows) * 256u);
            }
            if (live) {
                fence_proxy_async_smem();                // last tile's reads of the slot precede the new copy
                bulk_g2s(smem_u32(slot), p.wb + obase, 128u, wbfull);
            }

            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.f;

            for (int g = 0; g < ng; ++g, ++it) {
                const uint32_t a = it & 1, aph = (it >> 1) & 1;
                wait_bounded(tfull0 + 8 * a, aph, abort_flag, p.status, 3);
                tc_fence_after();
                const float u = su[g * RC_TILE + row];
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + a * RC_TILE + ch * 32, v);
                    tmem_ld_wait();
                    if (ch == 1) {                       // accumulator stage is in registers: hand it back
                        tc_fence_before();
                        mbar_arrive(tempty0 + 8 * a);
                    }
                    const float4* svp = reinterpret_cast<const float4*>(sv + g * RC_TILE + hh * 64 + ch * 32);
#pragma unroll
                    for (int i4 = 0; i4 < 8; ++i4) {
                        const float4 f = svp[i4];
                        const float vv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int i = i4 * 4 + j;
                            // exact int -> float for |P| < 2^22: 1.5 * 2^23 + P has P in its mantissa
                            const float pf = __fsub_rn(__int_as_float(static_cast<int>(v[i]) + 0x4B400000), 12582912.0f);
                            const float s = __fmul_rn(u, vv[j]);
                            acc[ch * 32 + i] = __fadd_rn(acc[ch * 32 + i], __fmul_rn(pf, s));
                        }
                    }
                    if (DBG && live) {
                        int32_t* d = p.dbg + (static_cast<size_t>(g) * p.M + m) * p.N + n0 + hh * 64 + ch * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<int4*>(d + i) = make_int4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    }
                }
            }
            wait_bounded(wbfull, tcount & 1, abort_flag, p.status, 5);
            if (live) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(slot + j * 16);
                    const uint32_t wq[4] = {wv.x, wv.y, wv.z, wv.w};
                    uint32_t oq[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float b0 = __uint_as_float(wq[e] << 16);
                        const float b1 = __uint_as_float(wq[e] & 0xFFFF0000u);
                        const __nv_bfloat162 o = __floats2bfloat162_rn(__fadd_rn(b0, acc[j * 8 + 2 * e]),
                                                                       __fadd_rn(b1, acc[j * 8 + 2 * e + 1]));
                        oq[e] = *reinterpret_cast<const uint32_t*>(&o);
                    }
                    *reinterpret_cast<uint4*>(p.out + obase + j * 8) = make_uint4(oq[0], oq[1], oq[2], oq[3]);
                }
            }
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ unpack producers
        const int pt = threadIdx.x - RC_EPI_THREADS;
        const int c = pt & 3, rbase = pt >> 2;
        const int my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const int total = my_tiles * ng;
        ProdRegs cur, nxt;
        if (total > 0) prod_load(cur, p, ng, (blockIdx.x / tiles_n) << 7, (blockIdx.x % tiles_n) << 7, 0, rbase, c);
        for (int idx = 0; idx < total; ++idx) {
            if (idx + 1 < total) {
                const int tile = blockIdx.x + ((idx + 1) / ng) * gridDim.x;
                prod_load(nxt, p, ng, (tile / tiles_n) << 7, (tile % tiles_n) << 7, (idx + 1) % ng, rbase, c);
            }
            const uint32_t s = idx % RC_STAGES, ph = (idx / RC_STAGES) & 1;
            wait_bounded(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, 2);
            uint8_t* A = stage_base + s * RC_STAGE_BYTES;
            uint8_t* B = A + RC_TILE * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                unpack_store(A, rbase + 32 * i, c, cur.qa[i], cur.za[i]);
                unpack_store(B, rbase + 32 * i, c, cur.qb[i], cur.zb[i]);
            }
            fence_proxy_async_smem();
            mbar_arrive(full0 + 8 * s);
            cur = nxt;
        }
    } else {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
                for (int g = 0; g < ng; ++g, ++it) {
                    const uint32_t s = it % RC_STAGES, ph = (it / RC_STAGES) & 1;
                    const uint32_t a = it & 1, aph = (it >> 1) & 1;
                    wait_bounded(tempty0 + 8 * a, aph ^ 1, abort_flag, p.status, 4);
                    wait_bounded(full0 + 8 * s, ph, abort_flag, p.status, 1);
                    tc_fence_after();
                    const uint32_t sa = smem_u32(stage_base + s * RC_STAGE_BYTES);
                    const uint64_t ad = smem_desc_k_sw128(sa);
                    const uint64_t bd = smem_desc_k_sw128(sa + RC_TILE * 128);
#pragma unroll
                    for (int k = 0; k < 4; ++k)          // 32 bytes of K per MMA inside the 128-byte row
                        tc_mma_i8(tmem_base + a * RC_TILE, ad + 2 * k, bd + 2 * k, RC_IDESC, k > 0 ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);           // operand stage reusable once these MMAs retire
                    tc_commit(tfull0 + 8 * a);           // accumulator stage ready
                }
            }
        }
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 12) tmem_dealloc(tmem_base, RC_TMEM_COLS);
}

}  // namespace ade
