// CUDA-core kernels of the grouped int8 GEMM path:
//   * gmm_simt_kernel, swiglu_simt_kernel - complete operators for shapes the TMA path cannot take (K or N not a multiple of
//                          16 bytes, unaligned pointers).  The reference accepts such shapes (its own unit
//                          tests use K=5, N=10), so they run here on the GPU instead of being rejected.
//   * combine_init_kernel - the initial contents of the finalize-routing result (weighted shared-expert rows, zeros).
// plus the plan / launch glue shared by both paths (make_plan: path, tile shape, workspace layout; launch).
//
// Arithmetic follows gmm/grouped_matmul/op_kernel/grouped_matmul_quant_mixcore.h:248-315 and
// gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant.h:367-513 step for step: every fp32
// operation is separately rounded (no fused multiply-add), bf16 and fp16 casts round to nearest even.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "gmm_common.h"

namespace gmm {
namespace {

__device__ __forceinline__ float load_scale1(const void *p, int dtype, size_t i)
{
    if (dtype == kF32) return __ldg(reinterpret_cast<const float *>(p) + i);
    const uint16_t h = __ldg(reinterpret_cast<const uint16_t *>(p) + i);
    if (dtype == kBF16) return __uint_as_float((uint32_t)h << 16);
    return __half2float(__ushort_as_half(h));
}

// q = int8(rint(half(S * (1 / (amax / 127)))))  -- CastFp32ToInt8Template,
// gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant_utils.h:308-316; NaN -> 0, saturating.
__device__ __forceinline__ int quant1(float s, float rcp)
{
    const __half h = __float2half_rn(__fmul_rn(s, rcp));
    int q = __half2int_rn(h);
    return max(-128, min(127, q));
}

// Locate the group of row m.  Same row-range rules as the tensor-core scheduler (group_list semantics of
// gmm/grouped_matmul/op_kernel/grouped_matmul_utils.h:243-257, clipped to [0, M]).
__device__ int find_group(const int64_t *gl, int L, int type, int M, int m)
{
    long long prev = 0, run = 0;
    for (int g = 0; g < L; ++g) {
        const int v = (int)gl[g];
        long long start, rows;
        if (type == 0) { start = prev; rows = (long long)v - prev; prev = v; }
        else { start = run; rows = v; if (v > 0) run += v; }
        if (rows < 0) rows = 0;
        if (start < 0) { rows += start; start = 0; if (rows < 0) rows = 0; }
        if (start > M) { start = M; rows = 0; }
        if (start + rows > M) rows = M - start;
        if (m >= start && m < start + rows) return g;
    }
    return -1;
}

struct SimtParams {
    const int8_t *x, *w;
    const void *w_scale;
    int w_scale_dtype;
    const float *x_scale;
    const void *bias;
    int bias_dtype;
    const int64_t *gl;
    int gl_len, gl_type;
    int M, K, N;
    long long wsk, wsn;  // weight element (k, n) of a group sits at k*wsk + n*wsn ...
    int nz;              // ... unless the layout is FRACTAL_NZ: ((n/32 * K/16 + k/16) * 16 + k%16) * 32 + n%32
    int act_type, mode, out_f16;
    void *out0;
    float *out1;
    const long long *out_row_index;
    int combine, row_index_i32, scatter_add;
    const float *logit;
    const void *row_index;
    long long out_rows;
};

__device__ __forceinline__ long long w_offset(const SimtParams &p, int k, int n)
{
    if (p.nz) return (((long long)(n >> 5) * (p.K >> 4) + (k >> 4)) * 16 + (k & 15)) * 32 + (n & 31);
    return k * p.wsk + n * p.wsn;
}

// One CTA per row; threads stride over the output columns.
__global__ void __launch_bounds__(256) gmm_simt_kernel(const SimtParams p)
{
    __shared__ int s_g;
    const int m = blockIdx.x;
    if (threadIdx.x == 0) s_g = find_group(p.gl, p.gl_len, p.gl_type, p.M, m);
    __syncthreads();
    const int g = s_g;
    if (g < 0) return;
    const int8_t *xr = p.x + (size_t)m * p.K;
    const int8_t *wg = p.w + (size_t)g * p.K * p.N;
    const float xs = p.x_scale ? p.x_scale[m] : 1.0f;
    const size_t orow = p.out_row_index ? (size_t)p.out_row_index[m] : (size_t)m;
    for (int n = threadIdx.x; n < p.N; n += blockDim.x) {
        int acc = 0;
        for (int k = 0; k < p.K; ++k) acc += (int)xr[k] * (int)wg[w_offset(p, k, n)];
        if (p.bias_dtype == kI32) acc += reinterpret_cast<const int *>(p.bias)[(size_t)g * p.N + n];
        if (p.mode == kModeInt32) {
            reinterpret_cast<int *>(p.out0)[orow * p.N + n] = acc;
            continue;
        }
        float t = __fmul_rn(__int2float_rn(acc), load_scale1(p.w_scale, p.w_scale_dtype, (size_t)g * p.N + n));
        if (p.combine) {  // grouped_matmul_finalize_routing: weighted row added to / stored at row row_index[m]
            const long long dst = p.row_index_i32 ? (long long)reinterpret_cast<const int *>(p.row_index)[m]
                                                  : reinterpret_cast<const long long *>(p.row_index)[m];
            const float lg = p.logit ? p.logit[m] : 1.0f;
            t = __fmul_rn(t, p.logit ? (p.x_scale ? __fmul_rn(xs, lg) : lg) : xs);
            if (p.bias_dtype == kBF16) t = __fadd_rn(t, __fmul_rn(lg, load_scale1(p.bias, kBF16, (size_t)g * p.N + n)));
            if (dst >= 0 && dst < p.out_rows) {
                float *o = reinterpret_cast<float *>(p.out0) + (size_t)dst * p.N + n;
                if (p.scatter_add) atomicAdd(o, t);
                else *o = t;
            }
            continue;
        }
        if (p.x_scale) t = __fmul_rn(t, xs);
        if (p.bias_dtype == kBF16) t = __fadd_rn(t, load_scale1(p.bias, kBF16, (size_t)g * p.N + n));
        t = apply_activation(p.act_type, t);
        if (p.out_f16) reinterpret_cast<__half *>(p.out0)[orow * p.N + n] = __float2half_rn(t);
        else reinterpret_cast<__nv_bfloat16 *>(p.out0)[orow * p.N + n] = __float2bfloat16_rn(t);
    }
}

// One CTA per row; S for the whole row is held in shared memory (N/2 <= 5120 floats).
__global__ void __launch_bounds__(256) swiglu_simt_kernel(const SimtParams p)
{
    extern __shared__ float s_row[];
    __shared__ int s_g;
    __shared__ float s_red[8];
    const int m = blockIdx.x, H = p.N / 2;
    if (threadIdx.x == 0) s_g = find_group(p.gl, p.gl_len, 0, p.M, m);
    __syncthreads();
    const int g = s_g;
    if (g < 0) return;
    const int8_t *xr = p.x + (size_t)m * p.K;
    const int8_t *wg = p.w + (size_t)g * p.K * p.N;
    const float xs = p.x_scale[m];
    float amax = 0.0f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        int a0 = 0, a1 = 0;
        for (int k = 0; k < p.K; ++k) {
            const int xv = xr[k];
            a0 += xv * (int)wg[w_offset(p, k, j)];
            a1 += xv * (int)wg[w_offset(p, k, j + H)];
        }
        const float a = __fmul_rn(__fmul_rn(__int2float_rn(a0), xs), load_scale1(p.w_scale, p.w_scale_dtype, (size_t)g * p.N + j));
        const float b = __fmul_rn(__fmul_rn(__int2float_rn(a1), xs), load_scale1(p.w_scale, p.w_scale_dtype, (size_t)g * p.N + H + j));
        const float sw = __fdiv_rn(a, __fadd_rn(1.0f, expf(-a)));
        const float s = __fmul_rn(b, sw);
        s_row[j] = s;
        amax = fmaxf(amax, fabsf(s));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = s_red[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) amax = fmaxf(amax, s_red[i]);
    const float qs = __fdiv_rn(amax, 127.0f);
    const float rcp = __fdiv_rn(1.0f, qs);
    if (threadIdx.x == 0) p.out1[m] = qs;
    int8_t *qrow = reinterpret_cast<int8_t *>(p.out0) + (size_t)m * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) qrow[j] = (int8_t)quant1(s_row[j], rcp);
}

// Rows [shared_offset, shared_offset + shared_rows) of y start as float(shared_input) * weight, all other rows as 0.
__global__ void __launch_bounds__(256) combine_init_kernel(float4 *y, const uint2 *shared, long long n4, long long rows,
                                                           long long shared_offset, long long shared_rows, float weight)
{
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        float4 *dst = y + r * n4;
        if (r >= shared_offset && r < shared_offset + shared_rows) {
            const uint2 *src = shared + (r - shared_offset) * n4;
            for (long long c = threadIdx.x; c < n4; c += blockDim.x) {
                const uint2 b = __ldg(src + c);  // four bf16
                float4 v;
                v.x = __fmul_rn(__uint_as_float(b.x << 16), weight);
                v.y = __fmul_rn(__uint_as_float(b.x & 0xffff0000u), weight);
                v.z = __fmul_rn(__uint_as_float(b.y << 16), weight);
                v.w = __fmul_rn(__uint_as_float(b.y & 0xffff0000u), weight);
                dst[c] = v;
            }
        } else {
            for (long long c = threadIdx.x; c < n4; c += blockDim.x) dst[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
}

// The same for a result or shared rows that are not 16 / 8-byte aligned (a tensor view with a storage offset) or whose
// width is not a multiple of 4: one element per thread and step.
__global__ void __launch_bounds__(256) combine_init_scalar_kernel(float *y, const uint16_t *shared, long long n, long long rows,
                                                                  long long shared_offset, long long shared_rows, float weight)
{
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        float v = 0.0f;
        if (r >= shared_offset && r < shared_offset + shared_rows)
            v = __fmul_rn(__uint_as_float((uint32_t)__ldg(shared + (i - shared_offset * n)) << 16), weight);
        y[i] = v;
    }
}

}  // namespace

cudaError_t combine_init_launch(const Problem &p, cudaStream_t stream)
{
    if (p.out_rows <= 0 || p.N <= 0) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(p.out0) & 3) return cudaErrorInvalidValue;
    const int sms = device_sm_count();
    const long long cap = (long long)(sms > 0 ? sms : 1) * 8;
    const bool vec = p.N % 4 == 0 && !(reinterpret_cast<uintptr_t>(p.out0) & 15) && !(reinterpret_cast<uintptr_t>(p.shared_input) & 7);
    if (!vec) {
        const long long total = p.out_rows * p.N;
        long long blocks = (total + 255) / 256;
        if (blocks > cap) blocks = cap;
        combine_init_scalar_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<float *>(p.out0),
                                                                        reinterpret_cast<const uint16_t *>(p.shared_input), p.N, p.out_rows,
                                                                        p.shared_offset, p.shared_input ? p.shared_rows : 0, p.shared_weight);
        return cudaGetLastError();
    }
    const long long n4 = p.N / 4;
    long long blocks = p.out_rows;  // whole rows per block
    if (blocks > cap) blocks = cap;
    combine_init_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<float4 *>(p.out0), reinterpret_cast<const uint2 *>(p.shared_input),
                                                             n4, p.out_rows, p.shared_offset, p.shared_input ? p.shared_rows : 0,
                                                             p.shared_weight);
    return cudaGetLastError();
}

int device_sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
    }
    return cached[dev];
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

void make_plan(const Problem &p, Plan *plan)
{
    plan->path = sm100_shape_ok(p) ? kPathSm100 : kPathSimt;
    // CTA pairs halve the weight traffic per SM but waste up to 255 rows at the end of every group, so they are
    // used when groups are long on average.  GMM_B200_CTAS=1|2 overrides the choice (for measurements).
    const long long avg_rows = p.rows_per_group_hint > 0 ? p.rows_per_group_hint : (p.gl_len > 0 ? p.M / p.gl_len : 0);
    plan->ctas = avg_rows >= 384 ? 2 : 1;
    if (const char *e = getenv("GMM_B200_CTAS")) {
        if (e[0] == '1') plan->ctas = 1;
        if (e[0] == '2') plan->ctas = 2;
    }
    // A second launch with 128-row tiles for the trailing blocks pays only when there are many of them: about half of the
    // groups end in such a block, and their tiles should fill the GPU several times over (measured: with 32 groups it loses
    // 5-8 %).  GMM_B200_HYBRID=0|1 overrides.
    {
        const long long n_tiles = p.mode == kModeSwigluQuant ? (p.N / 2 + 127) / 128 : (p.N + 255) / 256;
        constexpr long long kPlanSms = 148;  // a B200; phase 1 is host only and does not ask the device
        plan->hybrid = plan->ctas == 2 && (long long)p.gl_len * n_tiles >= 16ll * kPlanSms;
    }
    if (const char *e = getenv("GMM_B200_HYBRID")) plan->hybrid = plan->ctas == 2 && e[0] != '0';
    plan->off_status = 0;
    plan->off_wave = 0;
    size_t off = 256;
    plan->off_amax = off;
    if (p.mode == kModeSwigluQuant && plan->path == kPathSm100) {
        off += align_up((size_t)p.M * 4, 256);
        plan->off_done = off;  // two words per row block of a tile; every group can add a partial block in each of two launches
        off += align_up(((size_t)(p.M + 127) / 128 + 2 * (size_t)p.gl_len + 2) * 8, 256);
        // one pacing counter per wave of the tile schedule; at most one wave per tile (a single unit)
        const size_t max_tiles = ((size_t)(p.M + 127) / 128 + (size_t)p.gl_len) * (size_t)((p.N / 2 + 127) / 128);
        if (max_tiles <= 262144) {
            plan->off_wave = off;
            off += align_up((max_tiles + 1) * 4, 256);
        }
        plan->zero_bytes = off;
        plan->off_stage = off;
        off += align_up((size_t)p.M * (size_t)(p.N / 2) * 4, 256);
    } else {
        plan->zero_bytes = off;
        plan->off_stage = off;
    }
    plan->ws_bytes = off;
    plan->maps_ready = false;
}

cudaError_t simt_launch(const Problem &p, Plan &, void *, cudaStream_t stream)
{
    SimtParams sp;
    sp.x = p.x; sp.w = p.w; sp.w_scale = p.w_scale; sp.w_scale_dtype = p.w_scale_dtype; sp.x_scale = p.x_scale;
    sp.bias = p.bias; sp.bias_dtype = p.bias ? p.bias_dtype : kNone;
    sp.gl = p.group_list; sp.gl_len = p.gl_len; sp.gl_type = p.gl_type;
    sp.M = (int)p.M; sp.K = (int)p.K; sp.N = (int)p.N;
    sp.wsk = p.w_layout == 1 ? 1 : p.N;
    sp.wsn = p.w_layout == 1 ? p.K : 1;
    sp.nz = p.w_layout == 2;
    sp.act_type = p.act_type; sp.mode = p.mode; sp.out_f16 = p.out_f16; sp.out0 = p.out0; sp.out1 = reinterpret_cast<float *>(p.out1);
    sp.out_row_index = reinterpret_cast<const long long *>(p.out_row_index);
    sp.combine = p.combine; sp.row_index_i32 = p.row_index_i32; sp.scatter_add = p.scatter_add;
    sp.logit = p.logit; sp.row_index = p.row_index; sp.out_rows = p.out_rows;
    if (p.M <= 0) return cudaSuccess;
    if (p.mode == kModeSwigluQuant) {
        const size_t smem = (size_t)(p.N / 2) * sizeof(float);
        swiglu_simt_kernel<<<(int)p.M, 256, smem, stream>>>(sp);
    } else {
        gmm_simt_kernel<<<(int)p.M, 256, 0, stream>>>(sp);
    }
    return cudaGetLastError();
}

cudaError_t launch(const Problem &p, Plan &plan, void *workspace, size_t workspace_bytes, cudaStream_t stream)
{
    if (workspace_bytes < plan.ws_bytes || (plan.ws_bytes && !workspace)) return cudaErrorInvalidValue;
    if (plan.zero_bytes) {
        cudaError_t e = cudaMemsetAsync(workspace, 0, plan.zero_bytes, stream);
        if (e != cudaSuccess) return e;
    }
    if (p.combine && p.scatter_add) {
        cudaError_t e = combine_init_launch(p, stream);
        if (e != cudaSuccess) return e;
    }
    if (plan.path == kPathSm100) return sm100_launch(p, plan, workspace, stream);
    return simt_launch(p, plan, workspace, stream);
}

}  // namespace gmm
