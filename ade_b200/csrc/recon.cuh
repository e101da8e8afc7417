// Reconstructed application  W' = W_b + sum_g (us (x) vs) * P_g,  P_g = <Ucode - uz, Vcode - vz> over
// the 128 ranks of group g, contracted exactly in INT32 on the 5th-generation tensor cores.
//
// Replaces ade_recon_int4_kernel (src/kernels.py:262-381); arithmetic and rounding order are
// those of the reference's PyTorch statement of eq. (7) (src/quantization.py:303-315) followed
// by the base add of src/serving.py:92.
//
// One persistent CTA per SM walks 128 x 128 output tiles.  Warp roles:
//   warps 0-15  epilogue: tcgen05.ld of P_g, float conversion, per-group rescale in FP32
//               registers (32 accumulators per thread, packed two per 64-bit register), base
//               add, bf16 store.  Warp w owns tensor-memory lanes 32*(w%4).. and columns 32*(w/4)..
//               Sixteen warps rather than eight with twice the registers: this stage is bound
//               by issue latency, and four warps per scheduler hide it where two do not.
//               The base tile comes in and the merged tile goes out through a shared-memory
//               tile buffer so that every global access is a full 128-byte line (a thread owns a
//               row of the accumulator, but a warp moves two whole rows per instruction).
//   warps 16-19 unpack: the nibble-packed codes arrive through a per-thread cp.async ring three
//               work items deep (global latency never stalls the ring), are expanded to signed
//               int8 with the zero-point subtracted and written as K-major 128-byte-swizzled
//               operand tiles.
//   warp  20    one thread issues 4 x tcgen05.mma.kind::i8 (M=128, N=128, K=32) per group and
//               commits to mbarriers; it also owns the tensor-memory allocation.
// Rings: 3 raw code items and 2 operand stages (32 KB each) in shared memory, 2 accumulator
// stages in tensor memory (128 columns each).  Every mbarrier wait is bounded: when it expires the
// kernel raises a shared abort flag, records a code in *status, lets every later wait fall
// through and still runs to its normal end (tensor memory is released, no trap).
#pragma once
#include "ptx.cuh"

namespace ade {

constexpr int RC_TILE = 128;
constexpr int RC_STAGES = 2;                            // int8 operand stages
constexpr int RC_STAGE_BYTES = 2 * RC_TILE * 128;       // A tile + B tile, 128 int8 per row
constexpr int RC_EPI_WARPS = 16;                        // 4 lane quadrants x 4 column slices
constexpr int RC_EPI_THREADS = RC_EPI_WARPS * 32;
constexpr int RC_CW = RC_TILE / (RC_EPI_WARPS / 4);     // accumulator columns per epilogue thread
constexpr int RC_MMA_WARP = RC_EPI_WARPS + 4;
constexpr int RC_PROD_THREADS = 128;
constexpr int RC_THREADS = RC_EPI_THREADS + RC_PROD_THREADS + 32;
constexpr int RC_TMEM_COLS = 256;
constexpr int RC_RAW_DEPTH = 3;                         // raw code items in flight per unpack thread
constexpr int RC_RAW_ITEM = RC_PROD_THREADS * (8 * 16 + 8 * 4);   // per item: 8 x 16 B codes + 8 x 4 B zero words
constexpr long long RC_SPIN_LIMIT = 2000000000LL;       // default limit of a wait in clock cycles (about one second)
// instruction descriptor: D = S32 (bits 4-5 = 2), A = B = signed 8-bit (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 = 16 (bits 17-22), M >> 4 = 8 (bits 24-28)
// Every INT32 accumulator starts a group at the bit pattern of the float 1.5 * 2^23, so that after the
// integer MMAs its bits read as the float 1.5 * 2^23 + P (exact for |P| < 2^22; here |P| <= 28 800) and the
// int -> float conversion is one float subtraction.
constexpr uint32_t RC_MAGIC = 0x4B400000u;
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
    float one;      // 1.0f, set by the host: a value the assembler cannot fold (see recon_strip.cuh)
    long long spin_limit;   // clock cycles after which a wait gives up (RC_SPIN_LIMIT unless the host lowered it)
    int drop_loads;         // diagnostic: the code loads are not issued, so that the waits for them run out
    unsigned long long* trace;   // development builds (ADE_TRACE) only: event stamps of CTA 0, else nullptr
};

// Development aid, compiled out unless ADE_TRACE is defined: CTA 0 appends (code << 48 | clock) to one of a few
// tracks of 4096 stamps each; the host turns them into a timeline of the roles.
#ifdef ADE_TRACE
#define ADE_TRACE_STAMP(p, cnt, track, code)                                                                         \
    do {                                                                                                              \
        if ((p).trace && blockIdx.x == 0 && (cnt) < 4096)                                                             \
            (p).trace[(track) * 4096 + (cnt)++] = (static_cast<unsigned long long>(code) << 48) | (clock64() & 0xFFFFFFFFFFFFull); \
    } while (0)
#else
#define ADE_TRACE_STAMP(p, cnt, track, code) do { } while (0)
#endif

// what a bounded wait needs to give up: the CTA's abort flag, the caller's status word, the cycle limit
struct WaitCtx {
    volatile int* abort_flag;
    int* status;
    long long limit;
};

constexpr int RC_WB_ROW = 272;                          // one tile row: 256 bytes of bf16, padded (bank spread)
constexpr int RC_WB_BYTES = 2 * RC_TILE * RC_WB_ROW;    // two tile buffers (base in, merged out)

__host__ __device__ inline size_t recon_smem_bytes(int ng) {
    return 1024 /* alignment slack */ + static_cast<size_t>(RC_STAGES) * RC_STAGE_BYTES +
           static_cast<size_t>(RC_RAW_DEPTH) * RC_RAW_ITEM + RC_WB_BYTES +
           static_cast<size_t>(2) * ng * RC_TILE * (sizeof(float) + sizeof(uint16_t)) + 256;
}

__device__ __forceinline__ void wait_bounded(uint32_t bar, uint32_t parity, const WaitCtx& w, int code) {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(64);                                  // leave the issue slots to the warps that have work
        if (*w.abort_flag) return;
        if (clock64() - t0 > w.limit) {
            *w.abort_flag = 1;
            if (w.status) atomicCAS(w.status, 0, code);
            return;
        }
    }
}

// After an expired wait the roles run on without waiting for one another.  Before the CTA gives up its shared
// and tensor memory, let whatever is still in flight (tensor-map copies into shared memory, queued MMAs) land:
// a bounded sleep, far longer than any of them takes.
__device__ __forceinline__ void drain_after_abort(volatile int* abort_flag) {
    if (*abort_flag)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
}

// cp.async with zero fill: copies 16 (or 4) bytes when live, writes zeros otherwise
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4_zfill(uint32_t dst, const void* src, bool live) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(live ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// 32 packed codes (16 bytes) of operand row `row`, 16-byte column c of the packed row: expand to
// 32 signed bytes (code - zero) and store them as logical 16-byte chunks 2c, 2c+1 of the
// 128-byte row, XOR-swizzled with the row index as the 128-byte swizzle mode expects.
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

// Position of one unpack thread in the (tile, group) sequence of its CTA, with the addresses of
// the first of its four rows per operand (the other three are 32 rows further each).
struct ProdCursor {
    const uint8_t* ua;      // codes of U
    const uint8_t* vb;      // codes of V
    const uint8_t* uzp;     // zero-points of the U row
    const uint8_t* vzp;     // zero-points of the V column, group 0
    int tile, g, m_first;
};

__device__ __forceinline__ void cursor_set_tile(ProdCursor& c, const ReconParams& p, int ng, int tiles_n, int rbase,
                                                int cc) {
    const size_t rowb = static_cast<size_t>(p.r >> 1);
    const int m0 = (c.tile / tiles_n) << 7, n0 = (c.tile % tiles_n) << 7;
    c.m_first = m0 + rbase;
    c.ua = p.uq + static_cast<size_t>(c.m_first) * rowb + cc * 16;
    c.uzp = p.uz + static_cast<size_t>(c.m_first) * ng;
    c.vb = p.vq + static_cast<size_t>(n0 + rbase) * rowb + cc * 16;
    c.vzp = p.vz + n0 + rbase;
    c.g = 0;
}

// DBG = true additionally dumps every P_g to p.dbg (test builds of the launch only).
template <bool DBG>
__global__ void __launch_bounds__(RC_THREADS, 1) recon_kernel(const ReconParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int ng = p.r >> 7;
    uint8_t* stage_base = smem;
    uint8_t* raw_ring = smem + RC_STAGES * RC_STAGE_BYTES;                            // [RC_RAW_DEPTH][RC_RAW_ITEM]
    uint8_t* wb_stage = raw_ring + RC_RAW_DEPTH * RC_RAW_ITEM;                        // [2][128][272]
    float* sc = reinterpret_cast<float*>(wb_stage + RC_WB_BYTES);     // float32 [u|v][ng][128], then bf16 raw copy
    uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 3 * ng * RC_TILE);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8 * RC_STAGES;
    const uint32_t tfull0 = empty0 + 8 * RC_STAGES;
    const uint32_t tempty0 = tfull0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * RC_STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RC_STAGES; ++s) {
            mbar_init(full0 + 8 * s, RC_PROD_THREADS / 32);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull0 + 8 * a, 1);
            mbar_init(tempty0 + 8 * a, RC_EPI_WARPS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == RC_MMA_WARP) {
        tmem_alloc(smem_u32(tmem_slot), RC_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_n = p.N >> 7;
    const int ntiles = ((p.M + RC_TILE - 1) >> 7) * tiles_n;
    const WaitCtx wctx{abort_flag, p.status, p.spin_limit};

    if (warp < RC_EPI_WARPS) {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3, hh = warp >> 2;
        const int row = q * 32 + lane;
        const int et = threadIdx.x;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hh * RC_CW;
        const int crow = et >> 4, cck = et & 15;         // coalesced tile access: 16 threads per 256-byte row
        const int nsc = 2 * ng * RC_TILE;                // scale values per tile: [u | v][ng][128]
        float* su = sc;                                  // float32 scales of the current tile
        float* sv = sc + ng * RC_TILE;
        const uint16_t* raw_u = reinterpret_cast<const uint16_t*>(sc + nsc);          // bf16 [128 rows][ng], next tile
        const uint16_t* raw_v = raw_u + ng * RC_TILE;                                 // bf16 [ng][128]
        const uint32_t raw_s = smem_u32(raw_u);
        // Scales of a tile are two contiguous pieces of global memory per group at most: rows m0.. of us
        // (128 * ng values in one run) and 128 values of vs per group.  They are copied with cp.async
        // one tile ahead and converted to float32 at the start of their tile.
        auto issue_scales = [&](int tile) {
            if (tile < ntiles) {
                const int m0 = (tile / tiles_n) << 7, n0 = (tile % tiles_n) << 7;
                const int npieces = 32 * ng;             // 16-byte pieces: 16 * ng of us, then 16 per group of vs
                for (int j = et; j < npieces; j += RC_EPI_THREADS) {
                    if (j < 16 * ng) {
                        const long long off = (static_cast<long long>(m0) * ng) * 2 + j * 16;
                        const long long left = static_cast<long long>(p.M) * ng * 2 - off;
                        const int nbytes = left >= 16 ? 16 : (left > 0 ? static_cast<int>(left) : 0);
                        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.us) + (nbytes ? off : 0);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(raw_s + j * 16), "l"(src), "r"(nbytes)
                                     : "memory");
                    } else {
                        const int jj = j - 16 * ng, g = jj >> 4, piece = jj & 15;
                        cp_async16_zfill(raw_s + j * 16, p.vs + static_cast<size_t>(g) * p.N + n0 + piece * 8, true);
                    }
                }
            }
            cp_async_commit_group();
        };
        issue_scales(blockIdx.x);
        uint32_t magic4[4];                          // kept in four distinct registers (asm volatile: not merged)
#pragma unroll
        for (int i = 0; i < 4; ++i) asm volatile("mov.u32 %0, %1;" : "=r"(magic4[i]) : "n"(RC_MAGIC));
#pragma unroll
        for (int st = 0; st < 2; ++st)
#pragma unroll
            for (int ch = 0; ch < RC_CW / 16; ++ch) tmem_st16_fill(lane_addr + st * RC_TILE + ch * 16, magic4);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {                             // both accumulator stages start out armed and free
            mbar_arrive(tempty0);
            mbar_arrive(tempty0 + 8);
        }

        uint32_t it = 0, tcount = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
            const int m0 = (tile / tiles_n) << 7, n0 = (tile % tiles_n) << 7;
            const int m = m0 + row;
            const bool live = m < p.M;
            // base tile -> shared memory, two whole rows per warp instruction
            uint8_t* wbuf = wb_stage + (tcount & 1) * (RC_TILE * RC_WB_ROW);
            const uint32_t wbuf_s = smem_u32(wbuf);
#pragma unroll
            for (int j = 0; j < RC_TILE * 16 / RC_EPI_THREADS; ++j) {
                const int r_ = j * (RC_EPI_THREADS / 16) + crow;
                const bool lv = m0 + r_ < p.M;
                cp_async16_zfill(wbuf_s + r_ * RC_WB_ROW + cck * 16,
                                 p.wb + static_cast<size_t>(lv ? m0 + r_ : 0) * p.N + n0 + cck * 8, lv);
            }
            cp_async_commit_group();
            // scales of this tile were copied during the previous one: convert them to float32
            cp_async_wait_group<1>();                    // all but the base tile just issued
            asm volatile("bar.sync 1, %0;" ::"n"(RC_EPI_THREADS) : "memory");      // copies visible, old scales unused
            for (int e = et; e < nsc; e += RC_EPI_THREADS) {
                const int ee = e < ng * RC_TILE ? e : e - ng * RC_TILE;
                const int g = ee >> 7, i = ee & 127;
                su[e] = bf16_bits_to_f32(e < ng * RC_TILE ? raw_u[i * ng + g] : raw_v[g * RC_TILE + i]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(RC_EPI_THREADS) : "memory");      // float32 scales complete
            issue_scales(tile + gridDim.x);              // next tile's scales, consumed one tile later

            uint64_t acc[RC_CW / 2];                     // float32 accumulators as packed pairs
#pragma unroll
            for (int i = 0; i < RC_CW / 2; ++i) acc[i] = 0ull;
            const uint64_t neg_magic = f2_pack(-12582912.0f, -12582912.0f);

            for (int g = 0; g < ng; ++g, ++it) {
                const uint32_t a = it & 1, aph = (it >> 1) & 1;
                wait_bounded(tfull0 + 8 * a, aph, wctx, 3);
                tc_fence_after();
                const float u = su[g * RC_TILE + row];
                const uint64_t uu = f2_pack(u, u);
                const uint32_t tbase = lane_addr + a * RC_TILE;
                const ulonglong2* svp = reinterpret_cast<const ulonglong2*>(sv + g * RC_TILE + hh * RC_CW);
                // all of this thread's columns of the group, then the columns are re-armed and the accumulator stage is
                // handed back before any arithmetic
                uint32_t v[RC_CW / 16][16];
#pragma unroll
                for (int ch = 0; ch < RC_CW / 16; ++ch) tmem_ld16_sync(tbase + ch * 16, v[ch]);
#pragma unroll
                for (int ch = 0; ch < RC_CW / 16; ++ch) tmem_st16_fill(tbase + ch * 16, magic4);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * a);               // one arrival per warp
#pragma unroll
                for (int ch = 0; ch < RC_CW / 16; ++ch) {
                    const uint32_t (&vc)[16] = v[ch];
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const ulonglong2 f = svp[ch * 4 + i4];            // column scales of 4 columns
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int i = i4 * 4 + j * 2;
                            // the accumulator started at RC_MAGIC: its bits are the float 1.5 * 2^23 + P, exactly
                            const uint64_t pf = f2_add(f2_pack(__uint_as_float(vc[i]), __uint_as_float(vc[i + 1])), neg_magic);
                            const uint64_t s2 = f2_mul(uu, j == 0 ? f.x : f.y);      // us * vs, exact
                            acc[ch * 8 + i4 * 2 + j] = f2_add(acc[ch * 8 + i4 * 2 + j], f2_mul_rounded(pf, s2));
                        }
                    }
                    if (DBG && live) {
                        int32_t* d = p.dbg + (static_cast<size_t>(g) * p.M + m) * p.N + n0 + hh * RC_CW + ch * 16;
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            *reinterpret_cast<int4*>(d + i) = make_int4(vc[i] - RC_MAGIC, vc[i + 1] - RC_MAGIC, vc[i + 2] - RC_MAGIC,
                                                                        vc[i + 3] - RC_MAGIC);
                    }
                }
            }
            cp_async_wait_group<1>();                    // this thread's pieces of the base tile have landed
            asm volatile("bar.sync 1, %0;" ::"n"(RC_EPI_THREADS) : "memory");      // ... and everyone else's
            {
                uint8_t* own = wbuf + row * RC_WB_ROW + hh * (RC_CW * 2);  // this thread's row segment
#pragma unroll
                for (int j = 0; j < RC_CW / 8; ++j) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(own + j * 16);
                    const uint32_t wq[4] = {wv.x, wv.y, wv.z, wv.w};
                    uint32_t oq[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint64_t b2 = f2_pack(__uint_as_float(wq[e] << 16), __uint_as_float(wq[e] & 0xFFFF0000u));
                        float o0, o1;
                        f2_unpack(f2_add(b2, acc[j * 4 + e]), o0, o1);
                        const __nv_bfloat162 o = __floats2bfloat162_rn(o0, o1);
                        oq[e] = *reinterpret_cast<const uint32_t*>(&o);
                    }
                    *reinterpret_cast<uint4*>(own + j * 16) = make_uint4(oq[0], oq[1], oq[2], oq[3]);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(RC_EPI_THREADS) : "memory");      // merged tile complete
#pragma unroll
            for (int j = 0; j < RC_TILE * 16 / RC_EPI_THREADS; ++j) {
                const int r_ = j * (RC_EPI_THREADS / 16) + crow;
                if (m0 + r_ < p.M)
                    *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(m0 + r_) * p.N + n0 + cck * 8) =
                        *reinterpret_cast<const uint4*>(wbuf + r_ * RC_WB_ROW + cck * 16);
            }
        }
    } else if (warp < RC_MMA_WARP) {
        // ------------------------------------------------------------------ unpack producers
        const int pt = threadIdx.x - RC_EPI_THREADS;
        const int c = pt & 3, rbase = pt >> 2;
        const int my_tiles = static_cast<int>(blockIdx.x) < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const int total = p.drop_loads ? 0 : my_tiles * ng;   // diagnostic: no items, the MMA thread's wait runs out
        const size_t step = static_cast<size_t>(32) * (p.r >> 1);          // 32 rows further down a code array
        const uint32_t raw_s = smem_u32(raw_ring);
        ProdCursor ld, use;                               // issue position and consume position
        ld.tile = use.tile = blockIdx.x;
        if (total > 0) {
            cursor_set_tile(ld, p, ng, tiles_n, rbase, c);
            cursor_set_tile(use, p, ng, tiles_n, rbase, c);
        }
        auto advance = [&](ProdCursor& cur) {
            if (++cur.g == ng) {
                cur.tile += gridDim.x;
                if (cur.tile < ntiles) cursor_set_tile(cur, p, ng, tiles_n, rbase, c);
            }
        };
        // one work item (tile, group) = 8 x 16 bytes of codes and 8 aligned words holding the zero-points
        auto issue = [&](int idx) {
            if (idx < total) {
                const uint32_t base = raw_s + (idx % RC_RAW_DEPTH) * RC_RAW_ITEM;
                const uint32_t cs = base + pt * 16, zs = base + RC_PROD_THREADS * 128 + pt * 4;
                const int go = ld.g * 64;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const bool live = ld.m_first + 32 * i < p.M;           // rows past the matrix become zeros
                    const size_t off = live ? i * step : 0;
                    cp_async16_zfill(cs + i * (RC_PROD_THREADS * 16), ld.ua + off + go, live);
                    cp_async16_zfill(cs + (4 + i) * (RC_PROD_THREADS * 16), ld.vb + i * step + go, true);
                    const uint8_t* za = ld.uzp + (live ? static_cast<size_t>(32 * i) * ng : 0) + ld.g;
                    cp_async4_zfill(zs + i * (RC_PROD_THREADS * 4),
                                    reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(za) & ~uintptr_t(3)), live);
                    const uint8_t* zb = ld.vzp + static_cast<size_t>(ld.g) * p.N + 32 * i;
                    cp_async4_zfill(zs + (4 + i) * (RC_PROD_THREADS * 4),
                                    reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(zb) & ~uintptr_t(3)), true);
                }
                advance(ld);
            }
            cp_async_commit_group();                     // one group per item slot, empty past the end
        };
        for (int i = 0; i < RC_RAW_DEPTH - 1; ++i) issue(i);
        for (int idx = 0; idx < total; ++idx) {
            cp_async_wait_group<RC_RAW_DEPTH - 2>();     // item idx has landed
            const uint8_t* base = raw_ring + (idx % RC_RAW_DEPTH) * RC_RAW_ITEM;
            uint4 qa[4], qb[4];
            uint32_t za[4], zb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                qa[i] = *reinterpret_cast<const uint4*>(base + (i * RC_PROD_THREADS + pt) * 16);
                qb[i] = *reinterpret_cast<const uint4*>(base + ((4 + i) * RC_PROD_THREADS + pt) * 16);
                const uint32_t wa =
                    *reinterpret_cast<const uint32_t*>(base + RC_PROD_THREADS * 128 + (i * RC_PROD_THREADS + pt) * 4);
                const uint32_t wz =
                    *reinterpret_cast<const uint32_t*>(base + RC_PROD_THREADS * 128 + ((4 + i) * RC_PROD_THREADS + pt) * 4);
                const uint32_t sa = (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(use.uzp)) + 32u * i * ng + use.g) & 3u;
                const uint32_t sb = (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(use.vzp)) + 32u * i) & 3u;
                za[i] = (wa >> (8 * sa)) & 0xFFu;         // zero-filled words of dead rows give 0
                zb[i] = (wz >> (8 * sb)) & 0xFFu;
            }
            advance(use);
            issue(idx + RC_RAW_DEPTH - 1);               // refill the slot consumed one iteration ago
            const uint32_t s = idx % RC_STAGES, ph = (idx / RC_STAGES) & 1;
            wait_bounded(empty0 + 8 * s, ph ^ 1, wctx, 2);
            uint8_t* A = stage_base + s * RC_STAGE_BYTES;
            uint8_t* B = A + RC_TILE * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                unpack_store(A, rbase + 32 * i, c, qa[i], za[i]);
                unpack_store(B, rbase + 32 * i, c, qb[i], zb[i]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * s);   // one arrival per warp
        }
        cp_async_wait_group<0>();
    } else {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
                for (int g = 0; g < ng; ++g, ++it) {
                    const uint32_t s = it % RC_STAGES, ph = (it / RC_STAGES) & 1;
                    const uint32_t a = it & 1, aph = (it >> 1) & 1;
                    wait_bounded(tempty0 + 8 * a, aph, wctx, 4);   // use u of a stage waits for its u-th release
                    wait_bounded(full0 + 8 * s, ph, wctx, 1);
                    tc_fence_after();
                    const uint32_t sa = smem_u32(stage_base + s * RC_STAGE_BYTES);
                    const uint64_t ad = smem_desc_k_sw128(sa);
                    const uint64_t bd = smem_desc_k_sw128(sa + RC_TILE * 128);
#pragma unroll
                    for (int k = 0; k < 4; ++k)          // 32 bytes of K per MMA inside the 128-byte row
                        tc_mma_i8(tmem_base + a * RC_TILE, ad + 2 * k, bd + 2 * k, RC_IDESC, 1u);   // always on top of RC_MAGIC
                    tc_commit(empty0 + 8 * s);           // operand stage reusable once these MMAs retire
                    tc_commit(tfull0 + 8 * a);           // accumulator stage ready
                }
            }
        }
        __syncwarp();
    }

    drain_after_abort(abort_flag);
    tc_fence_before();
    __syncthreads();
    if (warp == RC_MMA_WARP) tmem_dealloc(tmem_base, RC_TMEM_COLS);
}

}  // namespace ade
