// C ABI of the B200 delta-application kernels (declared in include/ade_b200.h).
// Host side only validates arguments and launches; it never allocates or synchronises.
#include "../../include/ade_b200.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "compress.cuh"
#include "decode_ops.cuh"
#include "factored.cuh"
#include "recon.cuh"
#include "recon_strip.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

inline bool cuda_ok(cudaError_t e) {
    if (e != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(e);
        return false;
    }
    return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kMaxDevices = 64;
constexpr int kMaxRowsCap = 320;    // rows of one CTA's slice that fit the shared-memory y buffer (T = 128)
#ifndef ADE_FIFO_MIN
#define ADE_FIFO_MIN (400 * 1024)
#endif
constexpr size_t kFifoMinStream = ADE_FIFO_MIN;   // bytes of W_b per CTA from which the FIFO pays off at 9-16 tokens
constexpr int kMaxSmem = 232448;     // opt-in dynamic shared memory per CTA on sm_100
struct DeviceInfo {
    int ready = 0;      // 1 = usable, -1 = wrong architecture
    int sms = 0;
};
DeviceInfo g_dev[kMaxDevices];

// process-wide options (ade_b200_set_option)
long long g_wait_limit = ade::RC_SPIN_LIMIT;   // clock cycles a device-side wait may take before it gives up
int g_cooperative = 1;                         // factored kernel launched cooperatively (co-residency guaranteed)
int g_drop_signals = 0;                        // diagnostic: producers inside the kernels stay silent
int g_attn_single_pass = 1;                    // attention step: the single-pass kernel where the head dimension allows it
#ifdef ADE_TRACE
unsigned long long* g_trace = nullptr;         // development builds: device buffer for event stamps (option 100)
#endif

template <int NT>
bool optin_factored();

// per-device set-up: architecture check, SM count, dynamic shared-memory opt-in
int device_info(const DeviceInfo** out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return ADE_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return ADE_ERR_DEVICE;
    DeviceInfo& d = g_dev[dev];
    if (d.ready == 0) {
        int major = 0, sms = 0;
        if (!cuda_ok(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev))) return ADE_ERR_CUDA;
        if (!cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev))) return ADE_ERR_CUDA;
        if (major != 10) {
            d.ready = -1;
        } else {
            const int smem = kMaxSmem;
            if (!cuda_ok(cudaFuncSetAttribute(ade::recon_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) ||
                !cuda_ok(cudaFuncSetAttribute(ade::recon_strip_kernel<false, false, true, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
                return ADE_ERR_CUDA;
            if (!cuda_ok(cudaFuncSetAttribute(ade::compress_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              static_cast<int>(ade::compress_smem_bytes(ade::CQ_MAX_RANK, true)))))
                return ADE_ERR_CUDA;
            if (!optin_factored<1>() || !optin_factored<2>() || !optin_factored<4>() || !optin_factored<8>() ||
                !optin_factored<16>())
                return ADE_ERR_CUDA;
            d.sms = sms;
            d.ready = 1;
        }
    }
    if (d.ready < 0) return ADE_ERR_DEVICE;
    *out = &d;
    return ADE_OK;
}

// Tensor maps are encoded through the driver entry point, fetched once; the library does not link libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

bool load_encode_tiled() {
    if (g_encode_tiled) return true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (!cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q))) return false;
    if (q != cudaDriverEntryPointSuccess || !fn) return false;
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    return true;
}

// Row-major (outer x inner) array of `esize`-byte elements, contiguous rows.
bool make_map_2d(CUtensorMap* m, CUtensorMapDataType dt, int esize, const void* base, uint64_t inner, uint64_t outer,
                 uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * static_cast<uint64_t>(esize)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode_tiled(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = static_cast<int>(r);
        return false;
    }
    return true;
}

int check_delta(const ade_delta_t* d) {
    if (!d) return ADE_ERR_NULL;
    if (!d->uq || !d->us || !d->uz || !d->vs || !d->vz) return ADE_ERR_NULL;
    if (d->M < 1 || d->N < 1 || d->r < ADE_B200_GROUP || d->r > ADE_B200_MAX_RANK) return ADE_ERR_SHAPE;
    if (d->r % ADE_B200_GROUP || d->N % 128) return ADE_ERR_SHAPE;
    if (!aligned16(d->uq) || !aligned16(d->us) || !aligned16(d->uz) || !aligned16(d->vs) || !aligned16(d->vz))
        return ADE_ERR_ALIGN;
    return ADE_OK;
}

// ------------------------------------------------------------------ packing kernels
__global__ void pack_codes_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ out, int rows, int K,
                                  int transpose) {
    const size_t words = static_cast<size_t>(rows) * (K >> 3);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < words;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = i / (K >> 3);
        const int k0 = static_cast<int>(i % (K >> 3)) << 3;
        uint32_t c[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            c[j] = (transpose ? codes[static_cast<size_t>(k0 + j) * rows + row] : codes[row * K + k0 + j]) & 15u;
        // nibble order c0 c2 c4 c6 c1 c3 c5 c7
        out[i] = c[0] | (c[2] << 4) | (c[4] << 8) | (c[6] << 12) | (c[1] << 16) | (c[3] << 20) | (c[5] << 24) |
                 (c[7] << 28);
    }
}

__global__ void pack_zeros_kernel(const uint16_t* __restrict__ z, uint8_t* __restrict__ out, size_t count) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        out[i] = static_cast<uint8_t>(static_cast<int>(ade::bf16_bits_to_f32(z[i])));
}

// Rows per CTA: even split, minus `unit_rows` for each of the last CTAs that also computes 16 ranks of
// h = V^T x first.  That unit reads only about 5.5 rows' worth of bytes, but it costs one memory round trip
// under full load (4-5 us measured on 4096- and 11008-wide modules) before its own stream of W_b even
// starts; 14 rows is the compromise that helped every measured shape (a larger discount starves the
// other CTAs when many units exist, r = 512 has 32 of them).
void set_row_split(ade::FactoredParams& p, int grid) {
    const int n_units = p.r / 16;
    const int unit_ctas = n_units < grid ? n_units : grid;
    // side warps hide the unit at T <= 16; with sliced units (parts > 1) nearly every CTA owns one
    p.unit_rows = (p.w_b != nullptr && p.M / grid >= 24 && p.T > 16 && p.parts == 1) ? 14 : 0;
    const long long budget = static_cast<long long>(p.M) + static_cast<long long>(unit_ctas) * p.unit_rows;
    p.rows_cap = static_cast<int>(((budget + grid - 1) / grid + 1 + 31) / 32 * 32);
}

// The factored kernel's CTAs wait for one another (grid-wide counters), so the whole grid has to be resident at
// once.  A cooperative launch makes the driver guarantee that: the grid starts only when every CTA has an SM, also
// when other kernels occupy part of the device, and a grid that can never fit is refused at launch.
template <class Kernel>
int launch_grid(Kernel kernel, int grid, int threads, size_t smem, cudaStream_t st, const ade::FactoredParams& p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(threads));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_cooperative ? 1 : 0;
    return cuda_ok(cudaLaunchKernelEx(&cfg, kernel, p)) ? ADE_OK : ADE_ERR_CUDA;
}

// Launch of one of the small decode-step kernels.
template <class Kernel, class... Args>
int launch_small(Kernel kernel, int grid, int threads, size_t smem, void* stream, Args... args) {
    kernel<<<grid, threads, smem, static_cast<cudaStream_t>(stream)>>>(args...);
    return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
}

template <int NT, bool FUSE>
int launch_factored_one(ade::FactoredParams p, int grid, cudaStream_t st) {
    size_t smem = ade::factored_smem_bytes(NT, p.rows_cap, p.T, p.r);
    p.stages = 0;
    p.upf = 0;
    p.spin_limit = g_wait_limit;
    p.drop_arrivals = g_drop_signals;
    // Up to 8 tokens, or up to 16 with a long stream per CTA: W_b goes through a shared-memory FIFO (deeper than
    // registers allow).  At 9-16 tokens a short stream (a 4096 x 4096 module is 227 KB per CTA) is as fast with the
    // register prefetch: the deep FIFO raises the loaded memory latency, which the h hand-over pays several times.
    const size_t stream_bytes = static_cast<size_t>(p.M) * p.N * 2 / static_cast<size_t>(grid);
    if (FUSE && ade::fa_side(NT) && (NT == 1 || stream_bytes >= kFifoMinStream)) {
        const size_t room = (static_cast<size_t>(kMaxSmem) - smem) / ade::fa_fifo_item(NT);
        p.stages = room >= 2 ? static_cast<int>(room < static_cast<size_t>(ade::FA_FIFO_MAX) ? room : ade::FA_FIFO_MAX) : 0;
        smem += static_cast<size_t>(p.stages) * ade::fa_fifo_item(NT);
    }
    p.hstage = 0;
    if (!ade::fa_side(NT)) {                             // T > 16: h is staged in shared memory when it fits
        const size_t hs_bytes = ade::fa_side_region(p.T, p.r);
        if (smem + hs_bytes <= static_cast<size_t>(kMaxSmem)) {
            p.hstage = 1;
            smem += hs_bytes;
        }
    }
    // operands of the first phase-U items are prefetched into shared memory: the drained FIFO, or an area of their own
    // (not up to 8 tokens: there phase U runs on the side warps, under the stream of W_b, and needs no head start)
    if (ade::fa_side_u(NT)) {
        p.upf = 0;
    } else if (p.stages >= 2) {
        p.upf = ade::FA_UPF;
    } else if (smem + static_cast<size_t>(ade::FA_UPF) * ade::FA_UPF_ITEM <= static_cast<size_t>(kMaxSmem)) {
        p.upf = ade::FA_UPF;
        smem += static_cast<size_t>(ade::FA_UPF) * ade::FA_UPF_ITEM;
    }
    if constexpr (FUSE && ade::fa_side(NT)) {
        if (p.stages >= 2) {
            return launch_grid(ade::factored_kernel<NT, true, true>, grid, ade::fa_threads(NT), smem, st, p);
        }
    }
    return launch_grid(ade::factored_kernel<NT, FUSE>, grid, ade::fa_threads(NT), smem, st, p);
}

template <int NT>
int launch_factored(const ade::FactoredParams& p, int grid, cudaStream_t st) {
    return p.w_b ? launch_factored_one<NT, true>(p, grid, st) : launch_factored_one<NT, false>(p, grid, st);
}

template <int NT>
bool optin_factored() {
    if constexpr (ade::fa_side(NT)) {
        if (!cuda_ok(cudaFuncSetAttribute(ade::factored_kernel<NT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem)))
            return false;
    }
    return cuda_ok(cudaFuncSetAttribute(ade::factored_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem)) &&
           cuda_ok(cudaFuncSetAttribute(ade::factored_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem));
}

// block-diagonal hint of the delta -> kernel parameters (validated: ascending, covering [0, M) x [0, ng))
int set_blocks(ade::FactoredParams& p, const ade_delta_t* d) {
    p.n_blocks = 0;
    if (d->n_blocks == 0) return ADE_OK;
    if (d->n_blocks < 0 || d->n_blocks > ADE_B200_MAX_BLOCKS) return ADE_ERR_SHAPE;
    const int ng = d->r / ADE_B200_GROUP;
    if (d->block_rows[0] != 0 || d->block_groups[0] != 0 || d->block_rows[d->n_blocks] != d->M || d->block_groups[d->n_blocks] != ng)
        return ADE_ERR_SHAPE;
    for (int i = 0; i <= d->n_blocks; ++i) {
        if (i && (d->block_rows[i] <= d->block_rows[i - 1] || d->block_groups[i] <= d->block_groups[i - 1])) return ADE_ERR_SHAPE;
        p.block_rows[i] = d->block_rows[i];
        p.block_groups[i] = d->block_groups[i];
    }
    p.n_blocks = d->n_blocks;
    return ADE_OK;
}

// ---- scratch of ade_b200_factored_static: lives in the library image, one copy per GPU that loads it.
// Layout: 256 bytes of control words (words 0-3: the kernel's sync words, cleared before every launch; word 4:
// the status word, which only ade_b200_factored_static_status clears), always at the same place whatever T and
// r, then h = V^T x and, above 16 tokens, the partial sums of sliced phase-A units in what is left.  In host
// code this name is only a handle for cudaGetSymbolAddress.
__device__ __align__(256) unsigned char g_static_scratch[ADE_B200_STATIC_SCRATCH_BYTES];
void* g_static_scratch_addr[kMaxDevices] = {};

// Device address of the array on the current device; looked up on the first use per device.
int static_scratch_base(char** out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return ADE_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return ADE_ERR_DEVICE;
    if (g_static_scratch_addr[dev] == nullptr) {
        void* addr = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&addr, g_static_scratch)) || addr == nullptr) return ADE_ERR_CUDA;
        g_static_scratch_addr[dev] = addr;
    }
    *out = static_cast<char*>(g_static_scratch_addr[dev]);
    return ADE_OK;
}

}  // namespace

extern "C" {

int ade_b200_version(void) { return 1; }

int ade_b200_last_cuda_error(void) { return g_last_cuda_error; }

int ade_b200_device_status(void) {
    const DeviceInfo* di = nullptr;
    return device_info(&di);
}

int ade_b200_pack_codes(const uint8_t* codes, uint8_t* out, int rows, int K, int transpose, void* stream) {
    if (!codes || !out) return ADE_ERR_NULL;
    if (rows < 1 || K < 8 || K % 8) return ADE_ERR_SHAPE;
    if (!aligned16(out)) return ADE_ERR_ALIGN;
    const size_t words = static_cast<size_t>(rows) * (K >> 3);
    const int blocks = static_cast<int>((words + 255) / 256 < 65535 ? (words + 255) / 256 : 65535);
    pack_codes_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        codes, reinterpret_cast<uint32_t*>(out), rows, K, transpose);
    return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
}

int ade_b200_pack_zeros(const uint16_t* zeros_bf16, uint8_t* out, size_t count, void* stream) {
    if (!zeros_bf16 || !out) return ADE_ERR_NULL;
    if (count == 0) return ADE_OK;
    const int blocks = static_cast<int>((count + 255) / 256 < 65535 ? (count + 255) / 256 : 65535);
    pack_zeros_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(zeros_bf16, out, count);
    return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
}

// h: bf16 [T][r]; for T <= 16 two float32 partial sums [2][T][r] (each half of d_i is summed by another CTA);
// then the sync words.  This much is required.
static size_t factored_scratch_min(int T, int r) {
    const size_t b = static_cast<size_t>(T) * r * (T <= 16 ? 2 * sizeof(float) : sizeof(__nv_bfloat16));
    return ((b + 255) & ~static_cast<size_t>(255)) + 256;
}
// T > 16: slices of d_i per 16-rank unit of phase A, so that about 128 CTAs share it instead of r / 16
static int factored_parts_wanted(int T, int r) { return T <= 16 || r >= 2048 ? 1 : (2048 / r > 8 ? 8 : 2048 / r); }

size_t ade_b200_factored_scratch_bytes(int T, int r) {
    if (T < 1 || r < 1) return 0;
    const int parts = factored_parts_wanted(T, r);
    // recommended size: behind the sync words, float32 [parts][T][r] partial sums (T > 16)
    return factored_scratch_min(T, r) + (parts > 1 ? static_cast<size_t>(parts) * T * r * sizeof(float) : 0);
}

size_t ade_b200_factored_sync_offset(int T, int r) {
    if (T < 1 || r < 1) return 0;
    return factored_scratch_min(T, r) - 256;
}

// how many slices fit behind the sync words of a scratch buffer of `bytes` bytes (1 = unsplit units)
static int factored_parts(int T, int r, int N, size_t bytes, bool fused_base) {
    // With the base GEMM in the same launch the units stay whole: slicing would put phase A in front of every CTA's
    // stream of W_b instead of r / 16 of them (measured slower on 11008 x 4096 at T = 24-32).
    int parts = fused_base ? 1 : factored_parts_wanted(T, r);
    const int by_chunks = (N >> 7) / 8;                       // at least one 128-column chunk per warp and slice
    if (parts > by_chunks) parts = by_chunks;
    const size_t room = bytes - factored_scratch_min(T, r);
    const size_t per = static_cast<size_t>(T) * r * sizeof(float);
    if (static_cast<size_t>(parts) * per > room) parts = static_cast<int>(room / per);
    return parts < 2 ? 1 : parts;
}

int ade_b200_factored(const ade_delta_t* d, const void* x, const void* y_dense, const void* w_b, void* out,
                      void* scratch, size_t scratch_bytes, int T, void* stream) {
    int rc = check_delta(d);
    if (rc) return rc;
    if (!d->vt || !x || !out || !scratch) return ADE_ERR_NULL;
    if ((y_dense == nullptr) == (w_b == nullptr)) return ADE_ERR_NULL;      // exactly one base term
    if (T < 1 || T > ADE_B200_MAX_TOKENS) return ADE_ERR_SHAPE;
    if (!aligned16(d->vt) || !aligned16(x) || !aligned16(out) || !aligned16(scratch) ||
        (y_dense && !aligned16(y_dense)) || (w_b && !aligned16(w_b)))
        return ADE_ERR_ALIGN;
    if (scratch_bytes < factored_scratch_min(T, d->r)) return ADE_ERR_SCRATCH;
    const DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc) return rc;
    ade::FactoredParams p;
    p.w_b = static_cast<const __nv_bfloat16*>(w_b);
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.y_dense = static_cast<const __nv_bfloat16*>(y_dense);
    p.uq = d->uq;
    p.vt = d->vt;
    p.us = d->us;
    p.uz = d->uz;
    p.vs = d->vs;
    p.vz = d->vz;
    p.h = static_cast<__nv_bfloat16*>(scratch);
    p.sync = reinterpret_cast<unsigned int*>(static_cast<char*>(scratch) + ade_b200_factored_sync_offset(T, d->r));
    p.status = p.sync + 2;
    p.parts = factored_parts(T, d->r, d->N, scratch_bytes, w_b != nullptr);
    p.hpart = reinterpret_cast<float*>(static_cast<char*>(scratch) + factored_scratch_min(T, d->r));
    p.out = static_cast<__nv_bfloat16*>(out);
    p.T = T;
    p.M = d->M;
    p.N = d->N;
    p.r = d->r;
    rc = set_blocks(p, d);
    if (rc) return rc;
    const int grid = di->sms;                                   // one persistent CTA per SM, all co-resident
    set_row_split(p, grid);
    if (p.rows_cap > kMaxRowsCap) return ADE_ERR_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (T <= 8) return launch_factored<1>(p, grid, st);
    if (T <= 16) return launch_factored<2>(p, grid, st);
    if (T <= 32) return launch_factored<4>(p, grid, st);
    if (T <= 64) return launch_factored<8>(p, grid, st);
    return launch_factored<16>(p, grid, st);
}

int ade_b200_factored_static(const ade_delta_t* d, const void* x, const void* y_dense, const void* w_b, void* out,
                             int T, void* stream) {
    int rc = check_delta(d);
    if (rc) return rc;
    if (!d->vt || !x || !out) return ADE_ERR_NULL;
    if ((y_dense == nullptr) == (w_b == nullptr)) return ADE_ERR_NULL;      // exactly one base term
    if (T < 1 || T > ADE_B200_MAX_TOKENS) return ADE_ERR_SHAPE;
    if (!aligned16(d->vt) || !aligned16(x) || !aligned16(out) || (y_dense && !aligned16(y_dense)) ||
        (w_b && !aligned16(w_b)))
        return ADE_ERR_ALIGN;
    const size_t h_bytes = static_cast<size_t>(T) * d->r * (T <= 16 ? 2 * sizeof(float) : sizeof(__nv_bfloat16));
    if (256 + h_bytes > ADE_B200_STATIC_SCRATCH_BYTES) return ADE_ERR_SCRATCH;    // T * r beyond the built-in buffer
    const DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc) return rc;
    char* base = nullptr;
    rc = static_scratch_base(&base);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the array keeps whatever the previous call left: the four sync words must start at zero (the status word
    // behind them is sticky until ade_b200_factored_static_status clears it)
    if (!cuda_ok(cudaMemsetAsync(base, 0, 16, st))) return ADE_ERR_CUDA;
    ade::FactoredParams p;
    p.w_b = static_cast<const __nv_bfloat16*>(w_b);
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.y_dense = static_cast<const __nv_bfloat16*>(y_dense);
    p.uq = d->uq;
    p.vt = d->vt;
    p.us = d->us;
    p.uz = d->uz;
    p.vs = d->vs;
    p.vz = d->vz;
    p.sync = reinterpret_cast<unsigned int*>(base);
    p.status = p.sync + 4;
    p.h = reinterpret_cast<__nv_bfloat16*>(base + 256);
    {
        // what is left of the array behind h takes the partial sums of sliced phase-A units (T > 16)
        const size_t h_end = 256 + ((h_bytes + 255) & ~static_cast<size_t>(255));
        const size_t room = ADE_B200_STATIC_SCRATCH_BYTES > h_end ? ADE_B200_STATIC_SCRATCH_BYTES - h_end : 0;
        p.parts = factored_parts(T, d->r, d->N, factored_scratch_min(T, d->r) + room, w_b != nullptr);
        p.hpart = reinterpret_cast<float*>(base + h_end);
    }
    p.out = static_cast<__nv_bfloat16*>(out);
    p.T = T;
    p.M = d->M;
    p.N = d->N;
    p.r = d->r;
    rc = set_blocks(p, d);
    if (rc) return rc;
    const int grid = di->sms;
    set_row_split(p, grid);
    if (p.rows_cap > kMaxRowsCap) return ADE_ERR_SHAPE;
    if (T <= 8) return launch_factored<1>(p, grid, st);
    if (T <= 16) return launch_factored<2>(p, grid, st);
    if (T <= 32) return launch_factored<4>(p, grid, st);
    if (T <= 64) return launch_factored<8>(p, grid, st);
    return launch_factored<16>(p, grid, st);
}

int ade_b200_compress_rows(const float* x, const float* sqrt_s, uint8_t* codes, uint16_t* scale, uint16_t* zero, int rows,
                           int r, int rotate, int transposed, void* stream) {
    if (!x || !codes || !scale || !zero) return ADE_ERR_NULL;
    if (rows < 1 || r < ADE_B200_GROUP || r > ade::CQ_MAX_RANK || r % ADE_B200_GROUP) return ADE_ERR_SHAPE;
    if (rotate && (r & (r - 1))) return ADE_ERR_SHAPE;                  // the in-kernel rotation is the Hadamard transform
    if (transposed && !aligned16(codes)) return ADE_ERR_ALIGN;
    const DeviceInfo* di = nullptr;
    const int rc = device_info(&di);
    if (rc) return rc;
    const int blocks_wanted = (rows + ade::CQ_ROWS - 1) / ade::CQ_ROWS;
    const int grid = blocks_wanted < 8 * di->sms ? blocks_wanted : 8 * di->sms;
    const size_t smem = ade::compress_smem_bytes(r, transposed != 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    __nv_bfloat16* sc = reinterpret_cast<__nv_bfloat16*>(scale);
    __nv_bfloat16* zp = reinterpret_cast<__nv_bfloat16*>(zero);
    if (transposed) ade::compress_rows_kernel<true><<<grid, ade::CQ_THREADS, smem, st>>>(x, sqrt_s, codes, sc, zp, rows, r, rotate);
    else ade::compress_rows_kernel<false><<<grid, ade::CQ_THREADS, smem, st>>>(x, sqrt_s, codes, sc, zp, rows, r, rotate);
    return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
}

int ade_b200_rmsnorm(const void* x, const void* weight, void* out, int rows, int H, long long x_row_stride, float eps, void* stream) {
    if (!x || !weight || !out) return ADE_ERR_NULL;
    if (rows < 1 || H < 1 || x_row_stride < H) return ADE_ERR_SHAPE;
    return launch_small(ade::rmsnorm_kernel, rows, 256, 0, stream, static_cast<const __nv_bfloat16*>(x),
                        static_cast<const __nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(weight),
                        static_cast<__nv_bfloat16*>(nullptr), static_cast<__nv_bfloat16*>(out), H, x_row_stride, 0LL, eps);
}

int ade_b200_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out, void* out, int rows, int H,
                         long long x_row_stride, long long residual_row_stride, float eps, void* stream) {
    if (!x || !residual || !weight || !sum_out || !out) return ADE_ERR_NULL;
    if (rows < 1 || H < 1 || x_row_stride < H || residual_row_stride < H) return ADE_ERR_SHAPE;
    return launch_small(ade::rmsnorm_kernel, rows, 256, 0, stream, static_cast<const __nv_bfloat16*>(x),
                        static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight),
                        static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(out), H, x_row_stride, residual_row_stride, eps);
}

int ade_b200_rope(const void* q, const void* k, const void* cos_t, const void* sin_t, void* q_out, void* k_out, int B, int T, int q_heads,
                  int k_heads, int head_dim, long long q_row_stride, long long k_row_stride, long long cs_batch_stride, void* stream) {
    if (!q || !k || !cos_t || !sin_t || !q_out || !k_out) return ADE_ERR_NULL;
    if (B < 1 || T < 1 || q_heads < 1 || k_heads < 1 || head_dim < 2 || (head_dim & 1)) return ADE_ERR_SHAPE;
    const long long total = static_cast<long long>(B) * T * (q_heads + k_heads) * head_dim;
    const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    return launch_small(ade::rope_kernel, blocks, 256, 0, stream, static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                        static_cast<const __nv_bfloat16*>(cos_t), static_cast<const __nv_bfloat16*>(sin_t), static_cast<__nv_bfloat16*>(q_out),
                        static_cast<__nv_bfloat16*>(k_out), B, T, q_heads, k_heads, head_dim, q_row_stride, k_row_stride, cs_batch_stride);
}

int ade_b200_silu_mul(const void* gate, const void* up, void* out, int rows, int cols, long long gate_row_stride, long long up_row_stride,
                      void* stream) {
    if (!gate || !up || !out) return ADE_ERR_NULL;
    if (rows < 1 || cols < 1 || gate_row_stride < cols || up_row_stride < cols) return ADE_ERR_SHAPE;
    const long long total = static_cast<long long>(rows) * cols;
    const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    return launch_small(ade::silu_mul_kernel, blocks, 256, 0, stream, static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
                        static_cast<__nv_bfloat16*>(out), rows, cols, gate_row_stride, up_row_stride);
}

int ade_b200_attn_decode(const void* q, const void* k, const void* v, const void* cos_t, const void* sin_t, const void* mask, void* k_cache,
                         void* v_cache, long long* pos, unsigned int* ticket, void* out, int B, int q_heads, int k_heads, int head_dim, int cache_len,
                         long long q_row_stride, long long k_row_stride, long long v_row_stride, long long cs_batch_stride,
                         long long mask_row_stride, float scale, void* stream) {
    if (!q || !k || !v || !cos_t || !sin_t || !k_cache || !v_cache || !pos || !out) return ADE_ERR_NULL;
    if (B < 1 || q_heads < 1 || k_heads < 1 || q_heads % k_heads || cache_len < 1) return ADE_ERR_SHAPE;
    if (head_dim < 32 || head_dim > 256 || head_dim % 32) return ADE_ERR_SHAPE;
    if (!aligned16(k_cache) || !aligned16(v_cache)) return ADE_ERR_ALIGN;
    if (g_attn_single_pass) {
        // head dimensions 32 / 64 / 128 / 256: one streaming pass over the cache (any cache length)
        const __nv_bfloat16 *qp = static_cast<const __nv_bfloat16*>(q), *kp = static_cast<const __nv_bfloat16*>(k),
                            *vp = static_cast<const __nv_bfloat16*>(v), *cp = static_cast<const __nv_bfloat16*>(cos_t),
                            *sp = static_cast<const __nv_bfloat16*>(sin_t);
        __nv_bfloat16 *kcp = static_cast<__nv_bfloat16*>(k_cache), *vcp = static_cast<__nv_bfloat16*>(v_cache), *op = static_cast<__nv_bfloat16*>(out);
        const bool* mp = static_cast<const bool*>(mask);
#define ADE_ATTN_STREAM(CH)                                                                                                       \
    return launch_small(ade::attn_decode_stream_kernel<CH>, B * q_heads, 128, 0, stream, qp, kp, vp, cp, sp, mp, kcp, vcp, pos, ticket, op, \
                        q_heads, k_heads, cache_len, q_row_stride, k_row_stride, v_row_stride, cs_batch_stride, mask_row_stride, scale)
        if (head_dim == 32) ADE_ATTN_STREAM(4);
        if (head_dim == 64) ADE_ATTN_STREAM(8);
        if (head_dim == 128) ADE_ATTN_STREAM(16);
        if (head_dim == 256) ADE_ATTN_STREAM(32);
#undef ADE_ATTN_STREAM
    }
    const size_t smem = (static_cast<size_t>(7) * head_dim + cache_len) * sizeof(float);
    if (smem > 48 * 1024) return ADE_ERR_SHAPE;                           // cache lengths up to about 10 000 positions
    return launch_small(ade::attn_decode_kernel, B * q_heads, 128, smem, stream, static_cast<const __nv_bfloat16*>(q),
                        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), static_cast<const __nv_bfloat16*>(cos_t),
                        static_cast<const __nv_bfloat16*>(sin_t), static_cast<const bool*>(mask), static_cast<__nv_bfloat16*>(k_cache),
                        static_cast<__nv_bfloat16*>(v_cache), pos, ticket, static_cast<__nv_bfloat16*>(out), q_heads, k_heads, head_dim, cache_len,
                        q_row_stride, k_row_stride, v_row_stride, cs_batch_stride, mask_row_stride, scale);
}

int ade_b200_factored_static_status(int* dst, int clear, void* stream) {
    if (!dst) return ADE_ERR_NULL;
    char* base = nullptr;
    const int rc = static_scratch_base(&base);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!cuda_ok(cudaMemcpyAsync(dst, base + 16, sizeof(int), cudaMemcpyDefault, st))) return ADE_ERR_CUDA;
    if (clear && !cuda_ok(cudaMemsetAsync(base + 16, 0, sizeof(int), st))) return ADE_ERR_CUDA;
    return ADE_OK;
}

int ade_b200_set_option(int option, long long value) {
    switch (option) {
        case ADE_OPT_WAIT_LIMIT_CYCLES:
            if (value < 0) return ADE_ERR_SHAPE;
            g_wait_limit = value == 0 ? ade::RC_SPIN_LIMIT : value;
            return ADE_OK;
        case ADE_OPT_COOPERATIVE_LAUNCH:
            g_cooperative = value != 0;
            return ADE_OK;
        case ADE_OPT_DROP_SIGNALS:
            g_drop_signals = value != 0;
            return ADE_OK;
        case ADE_OPT_ATTN_SINGLE_PASS:
            g_attn_single_pass = value != 0;
            return ADE_OK;
#ifdef ADE_TRACE
        case 100:
            g_trace = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(value));
            return ADE_OK;
#endif
        default:
            return ADE_ERR_SHAPE;
    }
}

int ade_b200_expand_codes(const ade_delta_t* d, void* u8, void* v8, void* stream) {
    int rc = check_delta(d);
    if (rc) return rc;
    if (!d->vq || !u8 || !v8) return ADE_ERR_NULL;
    if (!aligned16(d->vq) || !aligned16(u8) || !aligned16(v8)) return ADE_ERR_ALIGN;
    const DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc) return rc;
    const int ng = d->r / ADE_B200_GROUP;
    const long long chunks = (static_cast<long long>(d->M) + d->N) * ng * 4;
    const long long want = (chunks + 255) / 256;
    const int grid = static_cast<int>(want < 8ll * di->sms ? want : 8ll * di->sms);
    ade::expand_codes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(d->uq, d->uz, d->vq, d->vz, static_cast<uint8_t*>(u8),
                                                                                 static_cast<uint8_t*>(v8), d->M, d->N, ng);
    return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
}

static int recon_impl(const ade_delta_t* d, const void* u8, const void* v8, const void* w_b, void* w_out, int32_t* dbg_acc,
                      int* status_dev, void* stream);

int ade_b200_recon(const ade_delta_t* d, const void* w_b, void* w_out, int32_t* dbg_acc, int* status_dev,
                   void* stream) {
    return recon_impl(d, nullptr, nullptr, w_b, w_out, dbg_acc, status_dev, stream);
}

int ade_b200_recon_expanded(const ade_delta_t* d, const void* u8, const void* v8, const void* w_b, void* w_out,
                            int32_t* dbg_acc, int* status_dev, void* stream) {
    if (!u8 || !v8) return ADE_ERR_NULL;
    if (!aligned16(u8) || !aligned16(v8)) return ADE_ERR_ALIGN;
    return recon_impl(d, u8, v8, w_b, w_out, dbg_acc, status_dev, stream);
}

static int recon_impl(const ade_delta_t* d, const void* u8, const void* v8, const void* w_b, void* w_out, int32_t* dbg_acc,
                      int* status_dev, void* stream) {
    int rc = check_delta(d);
    if (rc) return rc;
    if (!d->vq || !w_b || !w_out) return ADE_ERR_NULL;
    if (w_b == w_out) return ADE_ERR_NULL;
    if (!aligned16(d->vq) || !aligned16(w_b) || !aligned16(w_out) || (dbg_acc && !aligned16(dbg_acc)))
        return ADE_ERR_ALIGN;
    const DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc) return rc;
    ade::ReconParams p;
    p.uq = d->uq;
    p.vq = d->vq;
    p.us = d->us;
    p.uz = d->uz;
    p.vs = d->vs;
    p.vz = d->vz;
    p.wb = static_cast<const __nv_bfloat16*>(w_b);
    p.out = static_cast<__nv_bfloat16*>(w_out);
    p.dbg = dbg_acc;
    p.status = status_dev;
    p.M = d->M;
    p.N = d->N;
    p.r = d->r;
    p.one = 1.0f;
    p.spin_limit = g_wait_limit;
    p.drop_loads = g_drop_signals;
    p.trace = nullptr;
#ifdef ADE_TRACE
    p.trace = g_trace;
#endif
    const int ng = d->r / ADE_B200_GROUP;
    const int ntiles = ((d->M + ade::RC_TILE - 1) / ade::RC_TILE) * (d->N / ade::RC_TILE);
    const int grid = ntiles < di->sms ? ntiles : di->sms;
    if (ng <= ade::RS_MAX_GROUPS && ade::recon_strip_smem_bytes(ng, u8 != nullptr) <= static_cast<size_t>(kMaxSmem)) {
        // ranks up to 1024: the strip-resident kernel, all global traffic through tensor maps
        if (!load_encode_tiled()) return ADE_ERR_CUDA;
        ade::ReconMaps maps;
        const uint64_t M = static_cast<uint64_t>(d->M), N = static_cast<uint64_t>(d->N), rb = static_cast<uint64_t>(d->r / 2);
        if (!make_map_2d(&maps.wb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_b, N, M, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B) ||
            !make_map_2d(&maps.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_out, N, M, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B) ||
            !make_map_2d(&maps.uq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d->uq, rb, M, 64, 128, CU_TENSOR_MAP_SWIZZLE_NONE) ||
            !make_map_2d(&maps.vq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d->vq, rb, N, 64, 128, CU_TENSOR_MAP_SWIZZLE_NONE))
            return ADE_ERR_CUDA;
        const size_t smem = ade::recon_strip_smem_bytes(ng, u8 != nullptr);
        const cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (u8) {
            const uint64_t r = static_cast<uint64_t>(d->r);
            if (!make_map_2d(&maps.u8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, u8, r, M, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B) ||
                !make_map_2d(&maps.v8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, v8, r, N, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B))
                return ADE_ERR_CUDA;
            if (ng > 4) {
                if (dbg_acc) ade::recon_strip_kernel<true, true, true><<<grid, ade::RS_THREADS_EXP, smem, st>>>(p, maps);
                else ade::recon_strip_kernel<false, true, true><<<grid, ade::RS_THREADS_EXP, smem, st>>>(p, maps);
            } else {
                if (dbg_acc) ade::recon_strip_kernel<true, false, true><<<grid, ade::RS_THREADS_EXP, smem, st>>>(p, maps);
                else if (ng == 4) ade::recon_strip_kernel<false, false, true, 4><<<grid, ade::RS_THREADS_EXP, smem, st>>>(p, maps);
                else ade::recon_strip_kernel<false, false, true><<<grid, ade::RS_THREADS_EXP, smem, st>>>(p, maps);
            }
            return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
        }
        if (ng > 4) {
            if (dbg_acc) ade::recon_strip_kernel<true, true><<<grid, ade::RS_THREADS, smem, st>>>(p, maps);
            else ade::recon_strip_kernel<false, true><<<grid, ade::RS_THREADS, smem, st>>>(p, maps);
        } else {
            if (dbg_acc) ade::recon_strip_kernel<true, false><<<grid, ade::RS_THREADS, smem, st>>>(p, maps);
            else ade::recon_strip_kernel<false, false><<<grid, ade::RS_THREADS, smem, st>>>(p, maps);
        }
        return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
    }
    if (ade::recon_smem_bytes(ng) > static_cast<size_t>(kMaxSmem)) return ADE_ERR_SHAPE;    // rank too large for one CTA's scale tables
    if (dbg_acc)
        ade::recon_kernel<true><<<grid, ade::RC_THREADS, ade::recon_smem_bytes(ng), static_cast<cudaStream_t>(stream)>>>(p);
    else
        ade::recon_kernel<false><<<grid, ade::RC_THREADS, ade::recon_smem_bytes(ng), static_cast<cudaStream_t>(stream)>>>(p);
    return cuda_ok(cudaGetLastError()) ? ADE_OK : ADE_ERR_CUDA;
}

}  // extern "C"
