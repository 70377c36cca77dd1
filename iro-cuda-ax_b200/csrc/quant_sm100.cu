// Activation quantisation producer for the FP8 block-scaled GEMM: bf16 rows -> E4M3 bytes plus one
// fp32 scale per row per 128-wide K block (the 1x128 layout sA of axp_sm100_gemm_fp8_blockscaled).
//
//   amax  = max |x| over the block;  scale = amax / 448  (1 when the block is all zero)
//   q     = e4m3_satfinite_rne( x * (1 / scale) )
//
// Reference hooks: CastTile with the fp8_saturate policy (include/axp/protocol/convert/contracts.hpp:31,
// include/axp/detail/conversion.hpp:83-95).  The kernel is bound by HBM traffic (2 bytes read, 1 byte
// written per element): a lane moves 16 bytes in and 8 bytes out per step, a half-warp owns one
// 128-element block, the grid is a multiple of the SM count and strides over the blocks.
#include <cuda_bf16.h>

#include "axp/realize/sm100.hpp"
#include "host_common.hpp"

namespace rz = axp::realize::sm100;

namespace {

// Smallest block scale: the smallest normal float, so that 1 / scale stays finite (a block of denormal-sized values
// would otherwise give inv = inf and turn its exact zeros into NaN codes).
constexpr float kMinScale = 1.17549435e-38f;


constexpr int kQuantThreads = 256;

// Block scales of the up to 2 N blocks a warp has reduced (iteration i, half-warp h -> block 2 i + h): every lane of a
// half-warp holds its block maximum amax[i].  The two IEEE divisions per block (scale = amax / 448, inv = 1 / scale) are
// evaluated once per warp, by lane 2 i + h for block 2 i + h, and handed back by shuffles, instead of once per
// iteration by all lanes: the same operations on the same values, a quarter of the instructions for N = 4.
template <int N>
__device__ __forceinline__ void block_scales(const float (&amax)[N], int lane, float (&scale)[N], float (&inv)[N]) {
    static_assert(N >= 1 && N <= 4, "one lane per block: at most 8 blocks per warp");
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float a = __shfl_sync(0xffffffffu, amax[i], (lane & 1) * 16);      // block 2 i + (lane & 1)
        if ((lane >> 1) == i) mine = a;
    }
    const float sc = mine > 0.0f ? fmaxf(__fdiv_rn(mine, 448.0f), kMinScale) : 1.0f;
    const float iv = __fdiv_rn(1.0f, sc);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        scale[i] = __shfl_sync(0xffffffffu, sc, 2 * i + (lane >> 4));
        inv[i] = __shfl_sync(0xffffffffu, iv, 2 * i + (lane >> 4));
    }
}

// A warp handles a chunk of 8 consecutive blocks (1024 elements) of one row per step: four 16-byte loads per
// lane are issued before any arithmetic.  warps_x warps of a CTA sit side by side along the row, the other
// warps take further rows; CTAs stride over chunks (x) and rows (y).  No division in the loops.
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ X, uint8_t* __restrict__ Q, float* __restrict__ scales,
                          int M, int k_blocks, long long ldx, long long ldq, int warps_x) {
    const int lane = threadIdx.x & 31;
    const int half = lane >> 4;                 // which block of a pair
    const int l16 = lane & 15;                  // position inside the half-warp: elements [8*l16, 8*l16+8)
    const int warp = threadIdx.x >> 5;
    const int wx = warp % warps_x, wy = warp / warps_x;
    const int rows_per_cta = (kQuantThreads / 32) / warps_x;
    const int chunks = (k_blocks + 7) / 8;
    for (int m = blockIdx.y * rows_per_cta + wy; m < M; m += gridDim.y * rows_per_cta) {
        const __nv_bfloat16* xrow = X + (long long)m * ldx;
        uint8_t* qrow = Q + (long long)m * ldq;
        float* srow = scales + (long long)m * k_blocks;
        for (int chunk = blockIdx.x * warps_x + wx; chunk < chunks; chunk += gridDim.x * warps_x) {
            uint4 raw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kb = chunk * 8 + i * 2 + half;
                raw[i] = kb < k_blocks ? __ldg(reinterpret_cast<const uint4*>(xrow + kb * 128 + l16 * 8)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kb = chunk * 8 + i * 2 + half;
                const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
                float v[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[2 * e] = __uint_as_float(w[e] << 16);
                    v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                }
                float amax = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off, 16));
                // (sharing one division pair between the eight blocks of the step, as the RMSNorm kernel below does, costs
                // registers here and measured slower: this kernel is bound by HBM, not by issue slots)
                const float scale = amax > 0.0f ? fmaxf(__fdiv_rn(amax, 448.0f), kMinScale) : 1.0f;
                const float inv = __fdiv_rn(1.0f, scale);
                if (kb < k_blocks) {
                    uint2 out;
                    out.x = rz::PackE4m3x4::execute(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
                    out.y = rz::PackE4m3x4::execute(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
                    *reinterpret_cast<uint2*>(qrow + kb * 128 + l16 * 8) = out;
                    if (l16 == 0) srow[kb] = scale;
                }
            }
        }
    }
}

// RMSNorm fused with the quantiser: y = (x * inv_rms) * w, inv_rms = 1 / sqrt(mean(x^2) + eps), then the 1x128
// block quantisation above applied to y; the normalised row is never written.  Reference: RMSNorm fragment recipe
// (include/axp/level3/domain/norm.hpp:610-634: state, all-reduce, inv_rms, Mul by inv_rms, Mul by the weight) with
// inv_rms = rsqrt(mean_sq + eps) (norm.hpp:436-445).
// Persistent CTAs of 256 threads; a CTA takes rows blockIdx.x, blockIdx.x + gridDim.x, ...  Thread t holds elements
// [2048 c + 8 t, +8) of chunk c (K <= 16384) of the current row in registers, so x is read from HBM once; the weights are
// loaded once per CTA and stay in registers, and the next row of the CTA is requested before the current one is
// reduced, so that loads are in flight during the reduction and the arithmetic.  The sum of squares has a fixed order
// (so that the CPU oracle reproduces it bit for bit): per thread an fma chain over its elements in index order, an
// xor-butterfly over the warp (16, 8, 4, 2, 1), then the eight warp sums added left to right; sqrt and the divisions are
// IEEE.
constexpr int kNormThreads = 256;
constexpr int kNormMaxChunks = 8;

template <int kChunks>      // register chunks per thread: the smallest of 1, 2, 4, 8 that covers K / 2048
__global__ void __launch_bounds__(kNormThreads, kChunks <= 2 ? 3 : kChunks <= 4 ? 2 : 1)
rmsnorm_quantize_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, float eps,
                                  uint8_t* __restrict__ Q, float* __restrict__ scales, long long M, int K, long long ldx, long long ldq) {
    __shared__ float warp_sum[2][kNormThreads / 32];      // two sets: a fast warp may start the next row's reduction
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int l16 = lane & 15;
    auto load_row = [&](long long m, uint4 (&dst)[kChunks]) {
        const __nv_bfloat16* xrow = X + m * ldx;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int k0 = c * 2048 + t * 8;
            dst[c] = k0 < K ? __ldg(reinterpret_cast<const uint4*>(xrow + k0)) : make_uint4(0, 0, 0, 0);
        }
    };
    uint4 raw[kChunks], nxt[kChunks], wraw[kChunks];
    long long m = blockIdx.x;
    if (m < M) load_row(m, raw);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int k0 = c * 2048 + t * 8;
        wraw[c] = k0 < K ? __ldg(reinterpret_cast<const uint4*>(W + k0)) : make_uint4(0, 0, 0, 0);
    }
    for (int it = 0; m < M; ++it, m += gridDim.x) {
        const long long m_next = m + gridDim.x;
        if (m_next < M) load_row(m_next, nxt);
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
                ss = fmaf(lo, lo, ss);
                ss = fmaf(hi, hi, ss);
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
        float* sums = warp_sum[it & 1];
        if (lane == 0) sums[warp] = ss;
        __syncthreads();
        float total = sums[0];
#pragma unroll
        for (int i = 1; i < kNormThreads / 32; ++i) total = __fadd_rn(total, sums[i]);
        const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(K)), eps)));

        uint8_t* qrow = Q + m * ldq;
        float* srow = scales + m * (K / 128);
        // chunks in groups of up to four: a warp then holds up to eight block maxima, one division pair serves them all
        constexpr int kGroup = kChunks < 4 ? kChunks : 4;
#pragma unroll
        for (int c0 = 0; c0 < kChunks; c0 += kGroup) {
            float v[kGroup][8], amax[kGroup], scale[kGroup], inv[kGroup];
#pragma unroll
            for (int i = 0; i < kGroup; ++i) {
                const int c = c0 + i;
                const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
                const uint32_t ww[4] = {wraw[c].x, wraw[c].y, wraw[c].z, wraw[c].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[i][2 * e] = __fmul_rn(__fmul_rn(__uint_as_float(w[e] << 16), inv_rms), __uint_as_float(ww[e] << 16));
                    v[i][2 * e + 1] = __fmul_rn(__fmul_rn(__uint_as_float(w[e] & 0xffff0000u), inv_rms), __uint_as_float(ww[e] & 0xffff0000u));
                }
                float a = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(v[i][e]));
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off, 16));
                amax[i] = a;
            }
            block_scales<kGroup>(amax, lane, scale, inv);
#pragma unroll
            for (int i = 0; i < kGroup; ++i) {
                const int k0 = (c0 + i) * 2048 + t * 8;
                if (k0 < K) {
                    uint2 out;
                    out.x = rz::PackE4m3x4::execute(v[i][0] * inv[i], v[i][1] * inv[i], v[i][2] * inv[i], v[i][3] * inv[i]);
                    out.y = rz::PackE4m3x4::execute(v[i][4] * inv[i], v[i][5] * inv[i], v[i][6] * inv[i], v[i][7] * inv[i]);
                    *reinterpret_cast<uint2*>(qrow + k0) = out;
                    if (l16 == 0) srow[k0 / 128] = scale[i];
                }
            }
        }
#pragma unroll
        for (int c = 0; c < kChunks; ++c) raw[c] = nxt[c];
    }
}

}  // namespace

extern "C" int axp_sm100_rmsnorm_quantize_rows_e4m3(const void* X, const void* W, float eps, void* Q, float* scales, int64_t M,
                                                    int64_t K, int64_t ldx, int64_t ldq, void* stream) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_rmsnorm_quantize_rows_e4m3");
    using namespace axp_shim;
    if (!X || !W || !Q || !scales) return fail(AXP_ERR_BAD_ARG, "rmsnorm quantize: null pointer argument");
    if (M <= 0 || K <= 0) return fail(AXP_ERR_BAD_ARG, "rmsnorm quantize: M and K must be positive");
    if (K % 128 != 0) return fail(AXP_ERR_BAD_ARG, "rmsnorm quantize: K=%lld is not a multiple of the 128-wide scale block", (long long)K);
    if (K > 2048 * kNormMaxChunks) return fail(AXP_ERR_UNSUPPORTED, "rmsnorm quantize: K=%lld above %d (a row is held in registers)", (long long)K, 2048 * kNormMaxChunks);
    if (!(eps >= 0.0f)) return fail(AXP_ERR_BAD_ARG, "rmsnorm quantize: eps must be non-negative");
    if (ldx < K || ldq < K || ldx % 8 != 0 || ldq % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "rmsnorm quantize: leading dimensions must cover K and be multiples of 8 elements");
    if (!aligned16(X) || !aligned16(W) || (reinterpret_cast<uintptr_t>(Q) & 7u))
        return fail(AXP_ERR_BAD_ARG, "rmsnorm quantize: X and W must be 16-byte and Q 8-byte aligned");
    if (M > INT32_MAX / 2) return fail(AXP_ERR_UNSUPPORTED, "rmsnorm quantize: more than 2^30 rows");
    DeviceInfo dev;
    if (int rc = current_device_info(&dev); rc != AXP_OK) return rc;
    const int64_t chunks = (K + 2047) / 2048;
    // persistent grid: the CTAs that fit on the device at one time (or one per row, if there are fewer rows)
    const int64_t resident = int64_t(dev.sm_count) * (chunks <= 2 ? 3 : chunks <= 4 ? 2 : 1);
    const unsigned grid = unsigned(M < resident ? M : resident);
    auto launch = [&](auto kernel) {
        kernel<<<grid, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const __nv_bfloat16*>(X), static_cast<const __nv_bfloat16*>(W), eps, static_cast<uint8_t*>(Q), scales, (long long)M, int(K),
            ldx, ldq);
    };
    if (chunks <= 1) launch(rmsnorm_quantize_rows_e4m3_kernel<1>);
    else if (chunks <= 2) launch(rmsnorm_quantize_rows_e4m3_kernel<2>);
    else if (chunks <= 4) launch(rmsnorm_quantize_rows_e4m3_kernel<4>);
    else launch(rmsnorm_quantize_rows_e4m3_kernel<8>);
    AXP_CUDA_TRY(cudaGetLastError());
    return AXP_OK;
}

extern "C" int axp_sm100_quantize_rows_e4m3(const void* X, void* Q, float* scales, int64_t M, int64_t K, int64_t ldx,
                                            int64_t ldq, void* stream) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_quantize_rows_e4m3");
    using namespace axp_shim;
    if (!X || !Q || !scales) return fail(AXP_ERR_BAD_ARG, "quantize: null pointer argument");
    if (M <= 0 || K <= 0) return fail(AXP_ERR_BAD_ARG, "quantize: M and K must be positive");
    if (K % 128 != 0) return fail(AXP_ERR_BAD_ARG, "quantize: K=%lld is not a multiple of the 128-wide scale block", (long long)K);
    if (ldx < K || ldq < K || ldx % 8 != 0 || ldq % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "quantize: leading dimensions must cover K and be multiples of 8 elements");
    if (!aligned16(X) || (reinterpret_cast<uintptr_t>(Q) & 7u)) return fail(AXP_ERR_BAD_ARG, "quantize: X must be 16-byte and Q 8-byte aligned");
    DeviceInfo dev;
    if (int rc = current_device_info(&dev); rc != AXP_OK) return rc;
    if (M > INT32_MAX / 2 || K > INT32_MAX / 2) return fail(AXP_ERR_UNSUPPORTED, "quantize: extent above 2^30");
    const int k_blocks = int(K / 128);
    const int chunks = (k_blocks + 7) / 8;
    int warps_x = 1;
    while (warps_x * 2 <= chunks && warps_x * 2 <= kQuantThreads / 32) warps_x *= 2;
    const int rows_per_cta = (kQuantThreads / 32) / warps_x;
    const int grid_x = (chunks + warps_x - 1) / warps_x < 8 ? (chunks + warps_x - 1) / warps_x : 8;
    const int64_t row_ctas = (M + rows_per_cta - 1) / rows_per_cta;
    const int64_t cap_y = int64_t(dev.sm_count) * 8 / grid_x;                 // about 8 resident CTAs per SM
    const int grid_y = int(row_ctas < cap_y ? row_ctas : (cap_y > 0 ? cap_y : 1));
    quantize_rows_e4m3_kernel<<<dim3(unsigned(grid_x), unsigned(grid_y), 1), kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(X), static_cast<uint8_t*>(Q), scales, int(M), k_blocks, ldx, ldq, warps_x);
    AXP_CUDA_TRY(cudaGetLastError());
    return AXP_OK;
}
