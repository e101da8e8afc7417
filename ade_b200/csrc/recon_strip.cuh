// Reconstructed application for ranks up to 1024 (at most eight groups of 128): same arithmetic, same
// roundings and same tensor-core contraction as recon_kernel (recon.cuh), organised around a resident
// strip of the U operand.
//
// Replaces ade_recon_int4_kernel (src/kernels.py:262-381); arithmetic order of src/quantization.py:303-315,
// base add of src/serving.py:92.
//
// Every CTA owns a contiguous run of 128 x 128 output tiles in strip-major order (all n-tiles of a
// 128-row strip, then the next strip), so the expanded int8 form of the strip's U rows (128 x r bytes)
// is built once and stays in shared memory while only V tiles stream through.  All global traffic is
// tensor-map (TMA) traffic issued by single threads; no CTA-wide barrier exists after set-up.
//   warps 0-15  epilogue.  Warp w owns tensor-memory lanes 32*(w%4).. and 32 accumulator columns; it
//               loads its own 32 x 32 box of W_b with one TMA copy at the start of a tile, merges in
//               place and writes the box back with one TMA store.  Per group: tcgen05.ld, re-arm,
//               release, FP32 rescale as in recon.cuh.
//   warps 16-19 unpack: packed nibbles (raw ring filled by TMA) -> int8 minus zero-point, K-major
//               128-byte-swizzled operand tiles; U items go to the resident strip, V items to a ring.
//   warp  20    one thread issues tcgen05.mma.kind::i8 and the commits.
//   warp  21    one thread issues the TMA copies of packed codes and V zero-points (raw ring).
//   warp  22    scales: bf16 us / vs of the next tile -> float32 tables in shared memory (two buffers).
// Every mbarrier wait is bounded as in recon.cuh (abort flag, status word, normal exit).
//
// Expanded operands (template parameter EXP): when the caller has run expand_codes_kernel once (int8 code minus
// zero-point, (M + N) * r bytes), the load thread copies the operand tiles by TMA with the 128-byte swizzle straight
// into the resident strip and the V stages; the unpack role and the raw ring do not exist (19 warps, five V stages).
// The unpack warps were one of three roles that each needed about as long per group as the epilogue, and they
// took issue slots from it: gate_proj (11008 x 4096, r = 512) 75 -> 63 us per launch, same bits.
#pragma once
#include <cuda.h>

#include "recon.cuh"

namespace ade {

constexpr int RS_MAX_GROUPS = 8;                         // ranks up to 1024
constexpr int RS_EPI_WARPS = 16;
constexpr int RS_MMA_WARP = 20;
constexpr int RS_LOAD_WARP = 21;
constexpr int RS_SCALE_WARP = 22;
constexpr int RS_THREADS = 23 * 32;
// Expanded operands (int8 codes minus zero-point, prepared once by expand_codes_kernel): no unpack role, the operand
// tiles arrive by TMA in their 128-byte-swizzled form; the three single roles move down to warps 16-18.
constexpr int RS_THREADS_EXP = 19 * 32;
constexpr int RS_OPER_BYTES = RC_TILE * 128;             // one int8 operand tile of one group
constexpr int RS_RAW_CODES = RC_TILE * 64;               // 128 rows x 64 bytes of nibbles
constexpr int RS_RAW_SLOT = RS_RAW_CODES + 256;          // + 128 zero-points, padded
constexpr int RS_ACC_STAGES = 4;                        // 128-column accumulators in tensor memory (all 512 columns)
constexpr int RS_TMEM_COLS = RS_ACC_STAGES * RC_TILE;
constexpr int RS_BOX_BYTES = 32 * 64;                    // a warp's 32 x 32 bf16 box
// scale tables of one tile, per group: us of the 128 rows, then vs of the 128 columns, as float32
constexpr int RS_SC_BYTES = 512 + 512;

struct ReconMaps {
    CUtensorMap wb;     // (M, N) bf16, box 32 x 32, 64-byte swizzle
    CUtensorMap out;    // same geometry
    CUtensorMap uq;     // (M, r/2) bytes, box 128 rows x 64 bytes
    CUtensorMap vq;     // (N, r/2) bytes, box 128 rows x 64 bytes
    CUtensorMap u8;     // expanded operands only: (M, r) int8, box 128 rows x 128 bytes, 128-byte swizzle
    CUtensorMap v8;     // (N, r) int8, same box
};

// Ring depths and barrier indices.  BIG (five to eight groups): the resident strip takes up to 128 KB, so the
// rings shrink to two V stages, two raw slots and one box buffer per warp (measured: ring depth is not what
// limits this kernel).
template <bool BIG, bool EXP = false>
struct RsCfg {
    static constexpr int GROUPS = BIG ? 8 : 4;           // resident groups at most
    static constexpr int B_STAGES = EXP ? (BIG ? 3 : 5) : (BIG ? 2 : 3);   // int8 V tiles in flight
    static constexpr int RAW_DEPTH = EXP ? 1 : (BIG ? 2 : 4);                // packed items in flight (no ring when EXP)
    static constexpr int RAW_BYTES = EXP ? 0 : RAW_DEPTH * RS_RAW_SLOT;
    static constexpr int WB_BUFS = BIG ? 1 : 2;          // box buffers per epilogue warp
    static constexpr int WB_BYTES = RS_EPI_WARPS * WB_BUFS * RS_BOX_BYTES;
    // barrier indices (8 bytes each)
    static constexpr int BAR_RAW_FULL = 0;
    static constexpr int BAR_RAW_EMPTY = BAR_RAW_FULL + RAW_DEPTH;
    static constexpr int BAR_B_FULL = BAR_RAW_EMPTY + RAW_DEPTH;
    static constexpr int BAR_B_EMPTY = BAR_B_FULL + B_STAGES;
    static constexpr int BAR_A_FULL = BAR_B_EMPTY + B_STAGES;
    static constexpr int BAR_A_FREE = BAR_A_FULL + GROUPS;
    static constexpr int BAR_TFULL = BAR_A_FREE + 1;
    // Accumulators ready: with at most four groups a tile fits the four stages, and the issuer reports a whole tile
    // at once (barrier tile % 8: up to five tiles of a one-group delta are in flight); with more groups than stages
    // it reports every group (barrier = stage).
    static constexpr bool PER_TILE = EXP && !BIG;
    static constexpr int TFULL_BARS = 8;
    static constexpr int BAR_TEMPTY = BAR_TFULL + TFULL_BARS;
    static constexpr int BAR_SC_FULL = BAR_TEMPTY + RS_ACC_STAGES;
    static constexpr int BAR_SC_EMPTY = BAR_SC_FULL + 2;
    static constexpr int BAR_WB = BAR_SC_EMPTY + 2;
    static constexpr int BAR_COUNT = BAR_WB + WB_BUFS * RS_EPI_WARPS;
    __host__ __device__ static constexpr size_t smem_bytes(int ng) {
        return 1024 /* alignment slack */ + static_cast<size_t>(ng) * RS_OPER_BYTES + static_cast<size_t>(B_STAGES) * RS_OPER_BYTES +
               WB_BYTES + RAW_BYTES + static_cast<size_t>(ng) * RS_SC_BYTES * 2 + BAR_COUNT * 8 + 16;
    }
};

__host__ __device__ inline size_t recon_strip_smem_bytes(int ng, bool expanded = false) {
    if (expanded) return ng > 4 ? RsCfg<true, true>::smem_bytes(ng) : RsCfg<false, true>::smem_bytes(ng);
    return ng > 4 ? RsCfg<true>::smem_bytes(ng) : RsCfg<false>::smem_bytes(ng);
}

// As unpack_store (recon.cuh), with the tile given by its shared-window address.
__device__ __forceinline__ void unpack_store_s(uint32_t tile, int row, int c, uint4 q, uint32_t z) {
    const uint32_t zk = 0x80808080u - z * 0x01010101u;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = w[i] & 0x0F0F0F0Fu;
        const uint32_t hi = (w[i] >> 4) & 0x0F0F0F0Fu;
        o[2 * i] = (lo + zk) ^ 0x80808080u;
        o[2 * i + 1] = (hi + zk) ^ 0x80808080u;
    }
    const uint32_t rp = tile + row * 128;
    const int sw = row & 7;
    sts16(rp + (((2 * c) ^ sw) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    sts16(rp + (((2 * c + 1) ^ sw) << 4), make_uint4(o[4], o[5], o[6], o[7]));
}

// Packed codes -> int8 operands (code minus zero-point) in the byte order the unpack role of recon_strip_kernel
// produces: thread t turns the t-th 16-byte chunk of a (rows, r/2) code array into the t-th 32-byte chunk of the
// (rows, r) int8 array.  U zero-points are (M, ng) bytes, V zero-points (ng, N).
__global__ void __launch_bounds__(256) expand_codes_kernel(const uint8_t* __restrict__ uq, const uint8_t* __restrict__ uz,
                                                           const uint8_t* __restrict__ vq, const uint8_t* __restrict__ vz,
                                                           uint8_t* __restrict__ u8, uint8_t* __restrict__ v8, int M, int N, int ng) {
    const long long nu = static_cast<long long>(M) * ng * 4, total = nu + static_cast<long long>(N) * ng * 4;
    for (long long t = blockIdx.x * 256ll + threadIdx.x; t < total; t += gridDim.x * 256ll) {
        const bool is_u = t < nu;
        const long long e = is_u ? t : t - nu;
        const long long rg = e >> 2;                       // row * ng + group
        uint32_t z;
        if (is_u) {
            z = uz[rg];
        } else {
            const long long row = rg / ng;
            z = vz[(rg - row * ng) * N + row];
        }
        const uint4 q = *reinterpret_cast<const uint4*>((is_u ? uq : vq) + e * 16);
        const uint32_t zk = 0x80808080u - z * 0x01010101u;
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = ((w[i] & 0x0F0F0F0Fu) + zk) ^ 0x80808080u;
            o[2 * i + 1] = (((w[i] >> 4) & 0x0F0F0F0Fu) + zk) ^ 0x80808080u;
        }
        uint4* dst = reinterpret_cast<uint4*>((is_u ? u8 : v8) + e * 32);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// NG > 0: the number of groups is fixed at compile time (4: rank 512), so the epilogue's group loop unrolls with
// constant stage, table and tensor-memory offsets; 0: read from the delta.
template <bool DBG, bool BIG, bool EXP = false, int NG = 0>
__global__ void __launch_bounds__(EXP ? RS_THREADS_EXP : RS_THREADS, 1) recon_strip_kernel(const ReconParams p, const __grid_constant__ ReconMaps maps) {
    using C = RsCfg<BIG, EXP>;
    constexpr int MMA_WARP = EXP ? RS_EPI_WARPS : RS_MMA_WARP;
    constexpr int LOAD_WARP = MMA_WARP + 1;
    constexpr int SCALE_WARP = MMA_WARP + 2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw0 = smem_u32(smem_raw);
    const uint32_t base = (raw0 + 1023u) & ~1023u;
    const int ng = NG > 0 ? NG : (p.r >> 7);
    const uint32_t a_res = base;                                          // [ng][128][128] int8, resident strip of U
    const uint32_t b_st = a_res + ng * RS_OPER_BYTES;                     // [C::B_STAGES][128][128] int8
    const uint32_t wbuf = b_st + C::B_STAGES * RS_OPER_BYTES;             // [16 warps][2][32][64 B]
    const uint32_t rawr = wbuf + C::WB_BYTES;                             // [C::RAW_DEPTH][RS_RAW_SLOT]
    const uint32_t scf = rawr + C::RAW_BYTES;                             // [2][ng][RS_SC_BYTES] scale tables
    const uint32_t bars = scf + ng * RS_SC_BYTES * 2;
    uint8_t* gen = smem_raw + (bars - raw0);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + C::BAR_COUNT * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < C::RAW_DEPTH; ++i) {
            mbar_init(bar(C::BAR_RAW_FULL + i), 1);
            mbar_init(bar(C::BAR_RAW_EMPTY + i), 4);
        }
        for (int i = 0; i < C::B_STAGES; ++i) {
            mbar_init(bar(C::BAR_B_FULL + i), EXP ? 1 : 4);
            mbar_init(bar(C::BAR_B_EMPTY + i), 1);
        }
        for (int i = 0; i < C::GROUPS; ++i) mbar_init(bar(C::BAR_A_FULL + i), EXP ? 1 : 4);
        mbar_init(bar(C::BAR_A_FREE), 1);
        for (int i = 0; i < C::TFULL_BARS; ++i) mbar_init(bar(C::BAR_TFULL + i), 1);
        for (int i = 0; i < RS_ACC_STAGES; ++i) mbar_init(bar(C::BAR_TEMPTY + i), RS_EPI_WARPS);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(C::BAR_SC_FULL + i), 1);
            mbar_init(bar(C::BAR_SC_EMPTY + i), RS_EPI_WARPS);
        }
        for (int i = 0; i < C::WB_BUFS * RS_EPI_WARPS; ++i) mbar_init(bar(C::BAR_WB + i), 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(tmem_slot), RS_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_n = p.N >> 7;
    const int ntiles = ((p.M + RC_TILE - 1) >> 7) * tiles_n;
    const int t_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * ntiles / gridDim.x);
    const int t_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * ntiles / gridDim.x);
    const WaitCtx wctx{abort_flag, p.status, p.spin_limit};
    // first tile of this CTA as (strip, n-tile); every role then walks the tiles by incrementing (an integer division
    // per tile and role is a few hundred cycles of dependent instructions)
    const int strip0 = t_begin / tiles_n, nt0 = t_begin - strip0 * tiles_n;

    if (warp < RS_EPI_WARPS) {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3, hh = warp >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hh * 32;
        const uint32_t box0 = wbuf + warp * (C::WB_BUFS * RS_BOX_BYTES);
        const uint32_t own = lane * 64;                   // this thread's row of the box
        const int swz = (lane >> 1) & 3;                  // 64-byte swizzle: 16-byte chunk index ^ bits 7-8 of the address
        uint32_t magic4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) asm volatile("mov.u32 %0, %1;" : "=r"(magic4[i]) : "n"(RC_MAGIC));
#pragma unroll
        for (int st = 0; st < RS_ACC_STAGES; ++st)
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) tmem_st16_fill(lane_addr + st * RC_TILE + ch * 16, magic4);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int st = 0; st < RS_ACC_STAGES; ++st) mbar_arrive(bar(C::BAR_TEMPTY + st));
            prefetch_tensormap(&maps.wb);
            prefetch_tensormap(&maps.out);
        }

        uint32_t it = 0;
        bool tf_ready = false;                            // per-group barriers: the coming group's accumulator was seen complete
        int j = 0, sm = strip0, nt = nt0;
#ifdef ADE_TRACE
        int tcn = 0;
        const int ttrack = warp == 0 ? 0 : 1;
        const bool tr = (warp == 0 || warp == 9) && lane == 0;
#define EPI_STAMP(code) do { if (tr) ADE_TRACE_STAMP(p, tcn, ttrack, code); } while (0)
#else
#define EPI_STAMP(code) do { } while (0)
#endif
        for (int tile = t_begin; tile < t_end; ++tile, ++j) {
            const int m0 = sm << 7, n0 = nt << 7;
            const int m = m0 + row;
            EPI_STAMP(0x0100 | (j & 255));
            const bool live = m < p.M;
            const uint32_t b = j & 1, jph = (j >> 1) & 1;
            const uint32_t wbb = C::WB_BUFS == 2 ? b : 0, wph = C::WB_BUFS == 2 ? jph : static_cast<uint32_t>(j & 1);
            const uint32_t box = box0 + wbb * RS_BOX_BYTES;
            const uint32_t wbar = bar(C::BAR_WB + C::WB_BUFS * warp + wbb);
            // base box: with two buffers the box of tile j + 1 is requested during tile j (below), so only the CTA's first
            // tile asks here; with one buffer every tile asks for its own once the previous store has read the buffer
            if (lane == 0 && (C::WB_BUFS == 1 || j == 0)) {
                if (C::WB_BUFS == 1) bulk_wait_group_read<0>();
                mbar_arrive_expect_tx(wbar, RS_BOX_BYTES);
                tma_load_2d(box, &maps.wb, n0 + hh * 32, m0 + q * 32, wbar);
            }
            // A wait costs a few hundred cycles of this warp's time even when the phase completed long ago (a round
            // trip through shared memory and a branch, at this warp's share of the issue slots), so what a tile needs
            // is tested together, three tests in flight: scale tables, accumulators of the whole tile, base box
            // (requested a tile ago).  Only what is not there yet is waited for.
            const uint32_t tfb = bar(C::BAR_TFULL + (j & (C::TFULL_BARS - 1))), tfph = (j / C::TFULL_BARS) & 1;
            {
                const bool ok_sc = mbar_test(bar(C::BAR_SC_FULL + b), jph);
                const bool ok_tf = C::PER_TILE ? mbar_test(tfb, tfph) : true;
                const bool ok_wb = C::WB_BUFS == 2 ? mbar_test(wbar, wph) : true;
                if (!ok_sc) wait_bounded(bar(C::BAR_SC_FULL + b), jph, wctx, 5);
                if (!ok_tf) wait_bounded(tfb, tfph, wctx, 3);
                if (!ok_wb) wait_bounded(wbar, wph, wctx, 6);
            }
            if (C::PER_TILE) tc_fence_after();
            EPI_STAMP(0x0200 | (j & 255));
            const uint32_t sct = scf + b * (ng * RS_SC_BYTES);          // this tile's tables

            uint64_t acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0ull;
            const uint64_t one2 = f2_pack(p.one, p.one);  // 1.0f from the kernel parameters: acc + t as fma(t, 1, acc), never contracted

            // (Requesting the next 16-column chunk from tensor memory before rescaling the current one, across groups
            // too, was measured with the expanded operands: 61.8 us against 58.5 without.)
#pragma unroll(NG > 0 ? NG : 1)
            for (int g = 0; g < ng; ++g, ++it) {
                const uint32_t a = NG == RS_ACC_STAGES ? g : it % RS_ACC_STAGES, aph = (it / RS_ACC_STAGES) & 1;
                if (!C::PER_TILE) {
                    // the barrier of this group was tested while the previous group was being rescaled (a completed phase
                    // stays completed): the round trip of a wait is off the chain unless the accumulator really is late
                    if (!tf_ready) wait_bounded(bar(C::BAR_TFULL + a), aph, wctx, 3);
                    tc_fence_after();
                }
                EPI_STAMP(0x0300 | g);
                const uint32_t scg = sct + g * RS_SC_BYTES;
                const float u = __uint_as_float(lds4(scg + row * 4));
                const uint64_t uu = f2_pack(u, u);
                const float um = __fmul_rn(u, -12582912.0f);            // -m us, exact (m = 1.5 * 2^23)
                const uint64_t cc = f2_pack(um, um);
                const uint32_t tbase = lane_addr + a * RC_TILE;
                const uint32_t svg = scg + 512 + hh * 128;               // vs of this warp's 32 columns
                // The accumulator started at RC_MAGIC, so its bits are the float m + P, exactly.
                // x = fma(m + P, us, -m us) = P us exactly (|P| < 2^15, us has 8 significant bits);
                // t = x * vs is P * (us * vs) rounded once, as the reference rounds it; acc + t rounded once.
                auto rescale16 = [&](const uint32_t (&vc)[16], const int ch) {
#pragma unroll
                    for (int h4 = 0; h4 < 2; ++h4) {
                        uint64_t vs2[4];                 // vs of 8 columns as packed pairs, both loads in flight together
                        lds_f2x2(svg + (ch * 4 + h4 * 2) * 16, vs2[0], vs2[1]);
                        lds_f2x2(svg + (ch * 4 + h4 * 2 + 1) * 16, vs2[2], vs2[3]);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int k = h4 * 4 + kk;
                            const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(vc[2 * k]), __uint_as_float(vc[2 * k + 1])), uu, cc);
                            acc[ch * 8 + k] = f2_fma(f2_mul(x2, vs2[kk]), one2, acc[ch * 8 + k]);
                        }
                    }
                    if (DBG && live) {
                        int32_t* d = p.dbg + (static_cast<size_t>(g) * p.M + m) * p.N + n0 + hh * 32 + ch * 16;
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            *reinterpret_cast<int4*>(d + i) = make_int4(vc[i] - RC_MAGIC, vc[i + 1] - RC_MAGIC, vc[i + 2] - RC_MAGIC,
                                                                        vc[i + 3] - RC_MAGIC);
                    }
                };
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t vc[16];                     // 16 columns at a time: 32 would not fit the register budget
                    if (!C::PER_TILE && ch == 0) {       // is the next group's accumulator (next stage) there yet?  Used a group later.
                        const uint32_t a1 = (it + 1) % RS_ACC_STAGES, ph1 = ((it + 1) / RS_ACC_STAGES) & 1;
                        tf_ready = mbar_test(bar(C::BAR_TFULL + a1), ph1);
                    }
                    tmem_ld16_sync(tbase + ch * 16, vc);
                    EPI_STAMP(0x0400 | (g << 1) | ch);
                    tmem_st16_fill(tbase + ch * 16, magic4);             // re-arm, completes under the arithmetic
                    rescale16(vc, ch);
                }
                EPI_STAMP(0x0500 | g);
                tmem_st_wait();                          // accumulator stage re-armed: hand it back
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(C::BAR_TEMPTY + a));
                EPI_STAMP(0x0600 | g);
                if (C::WB_BUFS == 2 && g == 0 && lane == 0 && tile + 1 < t_end) {
                    // base box of the next tile into the other buffer; the store that last read it was issued a tile ago
                    const bool wrap = nt + 1 == tiles_n;
                    const uint32_t nb = b ^ 1;
                    const uint32_t nbar = bar(C::BAR_WB + C::WB_BUFS * warp + nb);
                    bulk_wait_group_read<0>();
                    mbar_arrive_expect_tx(nbar, RS_BOX_BYTES);
                    tma_load_2d(box0 + nb * RS_BOX_BYTES, &maps.wb, ((wrap ? 0 : nt + 1) << 7) + hh * 32, ((wrap ? sm + 1 : sm) << 7) + q * 32, nbar);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(C::BAR_SC_EMPTY + b));             // this warp is done with the scale tables
            EPI_STAMP(0x0700 | (j & 255));
            if (C::WB_BUFS == 1) wait_bounded(wbar, wph, wctx, 6);
            EPI_STAMP(0x0800 | (j & 255));
            uint4 wv4[4];                                // 8 columns per 16-byte chunk
#pragma unroll
            for (int c = 0; c < 4; ++c) wv4[c] = lds16(box + own + ((c ^ swz) << 4));
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t wq[4] = {wv4[c].x, wv4[c].y, wv4[c].z, wv4[c].w};
                uint32_t oq[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint64_t b2 = f2_pack(__uint_as_float(wq[e] << 16), __uint_as_float(wq[e] & 0xFFFF0000u));
                    float o0, o1;
                    f2_unpack(f2_add(b2, acc[c * 4 + e]), o0, o1);
                    const __nv_bfloat162 o = __floats2bfloat162_rn(o0, o1);
                    oq[e] = *reinterpret_cast<const uint32_t*>(&o);
                }
                sts16(box + own + ((c ^ swz) << 4), make_uint4(oq[0], oq[1], oq[2], oq[3]));
            }
            fence_proxy_async_smem();                    // merged box visible to the TMA store
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(&maps.out, n0 + hh * 32, m0 + q * 32, box);
                bulk_commit_group();
            }
            EPI_STAMP(0x0900 | (j & 255));
            if (++nt == tiles_n) {
                nt = 0;
                ++sm;
            }
        }
        if (lane == 0) bulk_wait_group_read<0>();    // shared memory may go once the last store has read it
    } else if (!EXP && warp < MMA_WARP) {
        // ------------------------------------------------------------------ unpack
        const int pt = threadIdx.x - RS_EPI_WARPS * 32;
        const int c = pt & 3, rbase = pt >> 2;
        uint32_t ri = 0, bi = 0, sk = 0;
        int cur_strip = -1;
#ifdef ADE_TRACE
        int tcn = 0;
#define UNP_STAMP(code) do { if (pt == 0) ADE_TRACE_STAMP(p, tcn, 2, code); } while (0)
#else
#define UNP_STAMP(code) do { } while (0)
#endif
        uint64_t za_pack[4] = {0, 0, 0, 0};               // zero-points of this thread's four U rows, one byte per group
        int sm = strip0, nt = nt0;
        for (int tile = t_begin; tile < t_end; ++tile) {
            const int strip = sm;
            if (++nt == tiles_n) {
                nt = 0;
                ++sm;
            }
            if (strip != cur_strip) {
                cur_strip = strip;
                const int m0 = strip << 7;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = m0 + rbase + 32 * i;
                    uint64_t z = 0;
                    if (m < p.M)
                        for (int g = 0; g < ng; ++g) z |= static_cast<uint64_t>(p.uz[static_cast<size_t>(m) * ng + g]) << (8 * g);
                    za_pack[i] = z;
                }
                if (sk > 0) wait_bounded(bar(C::BAR_A_FREE), (sk - 1) & 1, wctx, 7);   // old strip's MMAs retired
                for (int g = 0; g < ng; ++g, ++ri) {
                    const uint32_t slot = ri % C::RAW_DEPTH, ph = (ri / C::RAW_DEPTH) & 1;
                    wait_bounded(bar(C::BAR_RAW_FULL + slot), ph, wctx, 8);
                    const uint32_t rs = rawr + slot * RS_RAW_SLOT;
                    uint4 qa[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) qa[i] = lds16(rs + (rbase + 32 * i) * 64 + c * 16);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(C::BAR_RAW_EMPTY + slot));
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        unpack_store_s(a_res + g * RS_OPER_BYTES, rbase + 32 * i, c, qa[i], static_cast<uint32_t>(za_pack[i] >> (8 * g)) & 0xFFu);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(C::BAR_A_FULL + g));
                }
                ++sk;
            }
            for (int g = 0; g < ng; ++g, ++ri, ++bi) {
                const uint32_t slot = ri % C::RAW_DEPTH, ph = (ri / C::RAW_DEPTH) & 1;
                UNP_STAMP(0x1000 | g);
                wait_bounded(bar(C::BAR_RAW_FULL + slot), ph, wctx, 8);
                UNP_STAMP(0x1100 | g);
                const uint32_t rs = rawr + slot * RS_RAW_SLOT;
                uint4 qb[4];
                uint32_t zb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    qb[i] = lds16(rs + (rbase + 32 * i) * 64 + c * 16);
                    zb[i] = lds1(rs + RS_RAW_CODES + rbase + 32 * i);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(C::BAR_RAW_EMPTY + slot));
                const uint32_t s = bi % C::B_STAGES, bph = (bi / C::B_STAGES) & 1;
                wait_bounded(bar(C::BAR_B_EMPTY + s), bph ^ 1, wctx, 2);
                UNP_STAMP(0x1200 | g);
#pragma unroll
                for (int i = 0; i < 4; ++i) unpack_store_s(b_st + s * RS_OPER_BYTES, rbase + 32 * i, c, qb[i], zb[i]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(C::BAR_B_FULL + s));
                UNP_STAMP(0x1300 | g);
            }
        }
    } else {
    if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        // With expanded operands the whole warp walks the loop and waits and one elected lane issues: the loop stays
        // warp-uniform, so its counters, barrier addresses and descriptors can live in uniform registers (431 instead
        // of 648 cycles per group for the four MMAs and their commits).  With the unpack role present a single thread
        // runs the loop (the other form was slower there).
        // (two issuing threads taking alternate groups were tried with the expanded operands: no faster)
        if (EXP || lane == 0) {
            uint32_t it = 0, k = 0, s = 0, bph = 0;
#ifdef ADE_TRACE
            int tcn = 0;
#define MMA_STAMP(code) do { if (lane == 0) ADE_TRACE_STAMP(p, tcn, 3, code); } while (0)
#else
#define MMA_STAMP(code) do { } while (0)
#endif
            int nt = nt0;
            uint32_t jt = 0;
            for (int tile = t_begin; tile < t_end; ++tile, ++jt) {
                const bool first = tile == t_begin || nt == 0;
                const bool last = tile == t_end - 1 || nt + 1 == tiles_n;
                if (++nt == tiles_n) nt = 0;
                for (int g = 0; g < ng; ++g, ++it) {
                    const uint32_t a = it % RS_ACC_STAGES, aph = (it / RS_ACC_STAGES) & 1;
                    MMA_STAMP(0x2000 | g);
                    {
                        const bool ok_e = mbar_test(bar(C::BAR_TEMPTY + a), aph), ok_b = mbar_test(bar(C::BAR_B_FULL + s), bph);
                        if (!ok_e) wait_bounded(bar(C::BAR_TEMPTY + a), aph, wctx, 4);
                        MMA_STAMP(0x2100 | g);
                        if (!ok_b) wait_bounded(bar(C::BAR_B_FULL + s), bph, wctx, 1);
                    }
                    MMA_STAMP(0x2200 | g);
                    if (first) wait_bounded(bar(C::BAR_A_FULL + g), k & 1, wctx, 9);
                    tc_fence_after();
                    const uint64_t ad = smem_desc_k_sw128(a_res + g * RS_OPER_BYTES);
                    const uint64_t bd = smem_desc_k_sw128(b_st + s * RS_OPER_BYTES);
                    if (!EXP || elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            tc_mma_i8(tmem_base + a * RC_TILE, ad + 2 * kk, bd + 2 * kk, RC_IDESC, 1u);
                        tc_commit(bar(C::BAR_B_EMPTY + s));
                        if (!C::PER_TILE) tc_commit(bar(C::BAR_TFULL + a));
                        else if (g == ng - 1) tc_commit(bar(C::BAR_TFULL + (jt & (C::TFULL_BARS - 1))));
                        if (last && g == ng - 1) tc_commit(bar(C::BAR_A_FREE));    // the strip of U may be overwritten
                    }
                    if (EXP) __syncwarp();
                    MMA_STAMP(0x2300 | g);
                    if (++s == C::B_STAGES) {
                        s = 0;
                        bph ^= 1;
                    }
                }
                if (last) ++k;
            }
        }
        __syncwarp();
    } else if (EXP && warp == LOAD_WARP) {
        // ------------------------------------------------------------------ expanded operands -> strip and V stages
        if (lane == 0 && !p.drop_loads) {
            prefetch_tensormap(&maps.u8);
            prefetch_tensormap(&maps.v8);
            uint32_t bi = 0, sk = 0;
            int cur_strip = -1;
            int sm = strip0, nt = nt0;
            for (int tile = t_begin; tile < t_end; ++tile) {
                const int strip = sm, n0 = nt << 7;
                if (++nt == tiles_n) {
                    nt = 0;
                    ++sm;
                }
                if (strip != cur_strip) {
                    cur_strip = strip;
                    if (sk > 0) wait_bounded(bar(C::BAR_A_FREE), (sk - 1) & 1, wctx, 7);   // old strip's MMAs retired
                    for (int g = 0; g < ng; ++g) {
                        mbar_arrive_expect_tx(bar(C::BAR_A_FULL + g), RS_OPER_BYTES);
                        tma_load_2d(a_res + g * RS_OPER_BYTES, &maps.u8, g * 128, strip << 7, bar(C::BAR_A_FULL + g));
                    }
                    ++sk;
                }
                for (int g = 0; g < ng; ++g, ++bi) {
                    const uint32_t s = bi % C::B_STAGES, bph = (bi / C::B_STAGES) & 1;
                    wait_bounded(bar(C::BAR_B_EMPTY + s), bph ^ 1, wctx, 2);
                    mbar_arrive_expect_tx(bar(C::BAR_B_FULL + s), RS_OPER_BYTES);
                    tma_load_2d(b_st + s * RS_OPER_BYTES, &maps.v8, g * 128, n0, bar(C::BAR_B_FULL + s));
                }
            }
        }
        __syncwarp();
    } else if (warp == LOAD_WARP) {
        // ------------------------------------------------------------------ packed codes -> raw ring
        if (lane == 0 && !p.drop_loads) {                   // diagnostic drop_loads: nothing arrives, the waits run out
            prefetch_tensormap(&maps.uq);
            prefetch_tensormap(&maps.vq);
            uint32_t ri = 0;
            int cur_strip = -1;
#ifdef ADE_TRACE
            int tcn = 0;
#endif
            int sm = strip0, nt = nt0;
            for (int tile = t_begin; tile < t_end; ++tile) {
                const int strip = sm, n0 = nt << 7;
                if (++nt == tiles_n) {
                    nt = 0;
                    ++sm;
                }
                if (strip != cur_strip) {
                    cur_strip = strip;
                    for (int g = 0; g < ng; ++g, ++ri) {
                        const uint32_t slot = ri % C::RAW_DEPTH, ph = (ri / C::RAW_DEPTH) & 1;
                        wait_bounded(bar(C::BAR_RAW_EMPTY + slot), ph ^ 1, wctx, 10);
                        mbar_arrive_expect_tx(bar(C::BAR_RAW_FULL + slot), RS_RAW_CODES);
                        tma_load_2d(rawr + slot * RS_RAW_SLOT, &maps.uq, g * 64, strip << 7, bar(C::BAR_RAW_FULL + slot));
                    }
                }
                for (int g = 0; g < ng; ++g, ++ri) {
                    const uint32_t slot = ri % C::RAW_DEPTH, ph = (ri / C::RAW_DEPTH) & 1;
                    wait_bounded(bar(C::BAR_RAW_EMPTY + slot), ph ^ 1, wctx, 10);
                    ADE_TRACE_STAMP(p, tcn, 4, 0x3000 | g);
                    mbar_arrive_expect_tx(bar(C::BAR_RAW_FULL + slot), RS_RAW_CODES + 128);
                    tma_load_2d(rawr + slot * RS_RAW_SLOT, &maps.vq, g * 64, n0, bar(C::BAR_RAW_FULL + slot));
                    bulk_g2s(rawr + slot * RS_RAW_SLOT + RS_RAW_CODES, p.vz + static_cast<size_t>(g) * p.N + n0, 128,
                             bar(C::BAR_RAW_FULL + slot));
                }
            }
        }
        __syncwarp();
    } else if (warp == SCALE_WARP) {
        // ------------------------------------------------------------------ scale tables, one tile ahead
        int j = 0, sm = strip0, nt = nt0;
        for (int tile = t_begin; tile < t_end; ++tile, ++j) {
            const int m0 = sm << 7, n0 = nt << 7;
            if (++nt == tiles_n) {
                nt = 0;
                ++sm;
            }
            const uint32_t b = j & 1, jph = (j >> 1) & 1;
            const uint32_t sct = scf + b * (ng * RS_SC_BYTES);
            // us: rows m0.. of a (M, ng) array = 128 * ng consecutive bf16; vs: 128 consecutive bf16 per group
            constexpr int NV = C::GROUPS / 2;           // 16-byte vectors per lane: 16 * ng of each kind over 32 lanes
            uint4 vu[NV], vv[NV];
            const long long u_first = static_cast<long long>(m0) * ng, u_total = static_cast<long long>(p.M) * ng;
#pragma unroll
            for (int t = 0; t < NV; ++t) {
                const int vi = lane + 32 * t;             // 16-byte vector index, 16 * ng of each kind
                vu[t] = make_uint4(0, 0, 0, 0);
                vv[t] = make_uint4(0, 0, 0, 0);
                if (vi < 16 * ng) {
                    const long long e0 = u_first + 8 * vi;
                    if (e0 + 8 <= u_total) {
                        vu[t] = ldg16(p.us + e0);
                    } else {
                        uint32_t w[4] = {0, 0, 0, 0};
                        for (int e = 0; e < 8; ++e)
                            if (e0 + e < u_total) w[e >> 1] |= static_cast<uint32_t>(p.us[e0 + e]) << (16 * (e & 1));
                        vu[t] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    vv[t] = ldg16(p.vs + static_cast<size_t>(vi >> 4) * p.N + n0 + (vi & 15) * 8);
                }
            }
            wait_bounded(bar(C::BAR_SC_EMPTY + b), jph ^ 1, wctx, 11);
#pragma unroll
            for (int t = 0; t < NV; ++t) {
                const int vi = lane + 32 * t;
                if (vi < 16 * ng) {
                    const uint32_t wu[4] = {vu[t].x, vu[t].y, vu[t].z, vu[t].w};
                    const uint32_t wv[4] = {vv[t].x, vv[t].y, vv[t].z, vv[t].w};
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int eu = 8 * vi + e;        // element of the strip: row * ng + group
                        const int r_ = eu / ng, g_ = eu - r_ * ng;
                        const uint32_t hu = (e & 1) ? (wu[e >> 1] & 0xFFFF0000u) : (wu[e >> 1] << 16);
                        sts4(sct + g_ * RS_SC_BYTES + r_ * 4, hu);
                    }
                    const uint32_t dst = sct + (vi >> 4) * RS_SC_BYTES + 512 + (vi & 15) * 32;   // 8 columns of group vi / 16
                    sts16(dst, make_uint4(wv[0] << 16, wv[0] & 0xFFFF0000u, wv[1] << 16, wv[1] & 0xFFFF0000u));
                    sts16(dst + 16, make_uint4(wv[2] << 16, wv[2] & 0xFFFF0000u, wv[3] << 16, wv[3] & 0xFFFF0000u));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(C::BAR_SC_FULL + b));
        }
    }
    }

    drain_after_abort(abort_flag);
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, RS_TMEM_COLS);
}

}  // namespace ade
