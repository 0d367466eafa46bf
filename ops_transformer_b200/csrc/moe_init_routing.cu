// MoeInitRoutingV3 on the GPU: the producer of the grouped GEMM path's inputs.  From token rows x [n, h] and the top-k
// expert ids [n, k] it writes the rows grouped by expert (stable in pair order), optionally quantised per row to int8
// with a dynamic scale, the row map and the per-expert counts - exactly the x / per-token scale / group list that
// grouped_matmul_swiglu_quant and grouped_matmul consume.
//
// Follows moe/moe_init_routing_v3/op_kernel of the reference: the key-value sort of (expert id, pair index)
// (moe_v3_sort_*.h; equal keys keep their pair order), ExpertTokensCount (moe_v3_expert_tokens_count.h:246-282),
// RowIdxGather (moe_v3_row_idx_gather.h:141-156), MoeGatherOut (moe_v3_gather_out.h:197-233) and
// MoeGatherOutDynamicQuant::Compute (moe_v3_gather_dynamic_quant.h:103-143).
//
// Four launches, no host read in between:
//   count   - one histogram of the active experts per block of 1024 pairs
//   scan    - per expert (one CTA per 32 experts): exclusive prefix over the blocks; the CTA that finishes last then
//             scans over the experts: start of every expert's rows, the counts output, the number of rows
//   scatter - every pair finds its place: expert start + earlier blocks + earlier pairs of its block
//             (__match_any_sync ranks the lanes of a warp; the warps are ranked through a per-warp counter table, or take
//             turns when the active range is too wide for one), which keeps the order of equal keys
//   gather  - one CTA per token: the row is read once into registers, (quantised,) and stored at the output row of each
//             of its k pairs; shapes that do not fit the register tile take one CTA per output row
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "gmm_common.h"

namespace gmm {
namespace {

constexpr int kPairsPerBlock = 1024;

struct RoutingParams {
    const void *x;
    int x_dtype;               // kF32 / kF16 / kBF16 / kI8
    const int *expert_idx;     // [n, k]
    const float *scale;        // quant: smooth scale [range, h]; no quant: per-token scale [n]; may be null
    long long pairs;           // n * k
    int k, h;
    int e_start, range, expert_num;
    int quant, row_idx_type, count_type, vec_ok;
    void *expanded_x;
    int *expanded_row_idx;
    long long *counts_out;
    float *expanded_scale;
    int *block_hist;           // [nb, range]: pairs per block and active expert
    int *block_off;            // [nb, range]: the same, summed over the earlier blocks
    int *expert_first;         // [range]: first output row of every active expert
    int *sorted_row;           // [pairs]: pair index of every output row
    int *pair_pos;             // [pairs]: output row of every pair, -1 if its expert is not active
    int *total;                // number of output rows
    int nb;
};

// Programmatic dependent launch.  The kernels of one call form a chain (count -> scatter -> gather) in which the next
// kernel has work that does not depend on the previous one: the gather kernel loads and quantises its token before it needs
// the row positions.  A kernel that calls pdl_release() lets the next launch of the stream (if it was made with launch_pdl)
// start while this one still runs; that next kernel calls pdl_wait() before it touches anything this one writes, and the
// wait returns when this grid has ended and its writes are visible.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream, bool overlap,
                       Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

__global__ void __launch_bounds__(kPairsPerBlock) routing_count_kernel(const RoutingParams p)
{
    extern __shared__ int hist[];
    pdl_release();
    for (int e = threadIdx.x; e < p.range; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const long long j = (long long)blockIdx.x * kPairsPerBlock + threadIdx.x;
    if (j < p.pairs) {
        const int e = __ldg(p.expert_idx + j) - p.e_start;
        if (e >= 0 && e < p.range) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < p.range; e += blockDim.x) p.block_hist[(size_t)blockIdx.x * p.range + e] = hist[e];
    if (blockIdx.x == 0 && threadIdx.x == 0) p.total[1] = 0;  // arrival counter of the scan kernel that follows
}

// Inclusive scan of one int per thread over a 1024-thread block; returns the inclusive value, *block_sum the total.
__device__ int block_scan_1024(int v, int *warp_sums, int *block_sum)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int s = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += t;
        }
        warp_sums[lane] = s;
    }
    __syncthreads();
    if (warp > 0) v += warp_sums[warp - 1];
    *block_sum = warp_sums[31];
    __syncthreads();
    return v;
}

// Grid: one CTA per 32 active experts.  Part one (all CTAs): per expert the exclusive prefix over the blocks.  Part two
// (the CTA that arrives last at a counter; nobody waits): the scan over the experts and the counts output.
__global__ void __launch_bounds__(1024) routing_scan_kernel(const RoutingParams p)
{
    __shared__ int warp_sums[32];
    __shared__ int is_last;
    // per expert: exclusive prefix over the blocks, total into expert_first (as a count for now).  One warp per expert,
    // its lanes over 32 blocks at a time.
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int e = blockIdx.x * 32 + warp; e < min(p.range, (int)(blockIdx.x + 1) * 32); e += 32) {
            int carry = 0;
            for (int b0 = 0; b0 < p.nb; b0 += 32) {
                const int b = b0 + lane;
                const int t = b < p.nb ? p.block_hist[(size_t)b * p.range + e] : 0;
                int inc = t;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int u = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += u;
                }
                if (b < p.nb) p.block_off[(size_t)b * p.range + e] = carry + inc - t;
                carry += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (lane == 0) p.expert_first[e] = carry;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(p.total + 1, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // over the experts, 1024 at a time: first row of every expert, the counts output (count or key-value form)
    int row_carry = 0, nz_carry = 0;
    const int written_pairs = min(p.range + 1, p.expert_num);  // key-value form: entries the operator writes
    for (int base = 0; base < p.range; base += 1024) {
        const int e = base + threadIdx.x;
        const int c = e < p.range ? __ldcg(p.expert_first + e) : 0;  // written by other CTAs
        int sum_c, sum_nz;
        const int inc_c = block_scan_1024(c, warp_sums, &sum_c);
        const int inc_nz = block_scan_1024(c != 0 ? 1 : 0, warp_sums, &sum_nz);
        if (e < p.range) {
            p.expert_first[e] = row_carry + inc_c - c;
            if (p.count_type == 1) {
                p.counts_out[e] = c;
            } else if (c != 0) {
                const int slot = nz_carry + inc_nz - 1;
                p.counts_out[2 * (size_t)slot] = e + p.e_start;
                p.counts_out[2 * (size_t)slot + 1] = c;
            }
        }
        row_carry += sum_c;
        nz_carry += sum_nz;
    }
    if (p.count_type == 2)  // the compact list ends in zero entries (moe_v3_expert_tokens_count.h:126-128, 255-257)
        for (int i = nz_carry + threadIdx.x; i < written_pairs; i += blockDim.x) {
            p.counts_out[2 * (size_t)i] = 0;
            p.counts_out[2 * (size_t)i + 1] = 0;
        }
    if (threadIdx.x == 0) *p.total = row_carry;
}

constexpr int kWarpTableRange = 256;  // up to this many active experts the scatter keeps one counter per warp and expert

// PER_WARP: shared memory holds [32 warps][range] counters, all warps count at once and a scan over the warps gives every
// warp its start; otherwise one counter per expert and the warps take turns.
// FOLD (small tables: at most kWarpTableRange active experts and kFoldTable counters): the scan kernel is left out and
// every block derives what it needs from the block histograms itself - the rows of the earlier blocks and the first row
// of every expert - while block 0 also writes the counts output.  One launch less per call.
constexpr int kFoldTable = 8192;
template <bool PER_WARP, bool FOLD = false>
__global__ void __launch_bounds__(kPairsPerBlock) routing_scatter_kernel(const RoutingParams p)
{
    extern __shared__ int running[];
    __shared__ int s_first[FOLD ? kWarpTableRange : 1], s_off[FOLD ? kWarpTableRange : 1], s_tot[FOLD ? kWarpTableRange : 1];
    const int slots = PER_WARP ? p.range * (kPairsPerBlock / 32) : p.range;
    pdl_release();
    for (int e = threadIdx.x; e < slots; e += blockDim.x) running[e] = 0;
    pdl_wait();  // the block histograms (or the scan's tables) are complete
    if (FOLD) {
        __shared__ int warp_sums[32];
        for (int e = threadIdx.x; e < p.range; e += blockDim.x) {
            s_off[e] = 0;
            s_tot[e] = 0;
        }
        __syncthreads();
        // all threads share the table (one round trip to L2): per expert the total and the rows of the earlier blocks
        const int entries = p.nb * p.range;
        for (int i = threadIdx.x; i < entries; i += blockDim.x) {
            const int h = __ldg(p.block_hist + i);
            if (h != 0) {
                const int b = i / p.range, e = i - b * p.range;
                atomicAdd(&s_tot[e], h);
                if (b < (int)blockIdx.x) atomicAdd(&s_off[e], h);
            }
        }
        __syncthreads();
        // scan over the experts (range <= 256 <= blockDim): first row of every expert, and the counts output from block 0
        {
            const int e = threadIdx.x;
            const int c = e < p.range ? s_tot[e] : 0;
            int sum_c, sum_nz;
            const int inc_c = block_scan_1024(c, warp_sums, &sum_c);
            const int inc_nz = block_scan_1024(c != 0 ? 1 : 0, warp_sums, &sum_nz);
            if (e < p.range) s_first[e] = inc_c - c;
            if (blockIdx.x == 0) {  // in count or key-value form (as the scan kernel writes it)
                if (e < p.range) {
                    if (p.count_type == 1) {
                        p.counts_out[e] = c;
                    } else if (c != 0) {
                        p.counts_out[2 * (size_t)(inc_nz - 1)] = e + p.e_start;
                        p.counts_out[2 * (size_t)(inc_nz - 1) + 1] = c;
                    }
                }
                if (p.count_type == 2) {  // the compact list ends in zero entries (moe_v3_expert_tokens_count.h:126-128, 255-257)
                    const int written_pairs = min(p.range + 1, p.expert_num);
                    for (int i = sum_nz + threadIdx.x; i < written_pairs; i += blockDim.x) {
                        p.counts_out[2 * (size_t)i] = 0;
                        p.counts_out[2 * (size_t)i + 1] = 0;
                    }
                }
                if (threadIdx.x == 0) *p.total = sum_c;
            }
        }
    }
    const long long j = (long long)blockIdx.x * kPairsPerBlock + threadIdx.x;
    int e = -1;
    if (j < p.pairs) {
        e = __ldg(p.expert_idx + j) - p.e_start;
        if (e < 0 || e >= p.range) e = -1;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int before = 0;  // pairs of this block with the same expert that come earlier
    __syncthreads();
    if (PER_WARP) {
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && rank == 0) running[warp * p.range + e] = __popc(peers);
        __syncthreads();
        for (int x = threadIdx.x; x < p.range; x += blockDim.x) {  // exclusive scan over the warps, one expert per thread
            int run = 0;
#pragma unroll
            for (int w = 0; w < kPairsPerBlock / 32; ++w) {
                const int t = running[w * p.range + x];
                running[w * p.range + x] = run;
                run += t;
            }
        }
        __syncthreads();
        if (e >= 0) before = running[warp * p.range + e] + rank;
    } else {
        for (int w = 0; w < kPairsPerBlock / 32; ++w) {
            if (warp == w) {
                const unsigned peers = __match_any_sync(0xffffffffu, e);
                const int rank = __popc(peers & ((1u << lane) - 1u));
                int base = 0;
                if (e >= 0 && rank == 0) {
                    base = running[e];
                    running[e] = base + __popc(peers);
                }
                base = __shfl_sync(0xffffffffu, base, __ffs(peers) - 1);
                before = base + rank;
            }
            __syncthreads();
        }
    }
    if (j >= p.pairs) return;
    if (e < 0) {
        p.pair_pos[j] = -1;
        if (p.row_idx_type == 0) p.expanded_row_idx[j] = -1;
        return;
    }
    const int pos = FOLD ? s_first[e] + s_off[e] + before
                         : p.expert_first[e] + p.block_off[(size_t)blockIdx.x * p.range + e] + before;
    p.sorted_row[pos] = (int)j;
    p.pair_pos[j] = pos;
    if (p.row_idx_type == 1) p.expanded_row_idx[pos] = (int)j;
    else p.expanded_row_idx[j] = pos;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// fp32 -> fp16 towards zero, fp16 -> int8 to nearest with ties away from zero (CAST_TRUNC then CAST_ROUND,
// moe_v3_gather_dynamic_quant.h:134-137).  0 / 0 (an all-zero row) maps to 0.
__device__ __forceinline__ int8_t quant_trunc_round(float v, float scale)
{
    const float f = __half2float(__float2half_rz(__fdiv_rn(v, scale)));
    if (!(f == f)) return 0;
    const int q = (int)(f + (f < 0.0f ? -0.5f : 0.5f));
    return (int8_t)max(-128, min(127, q));
}

// One CTA per output row.  Dynamic quantisation: v = float(x) [* smooth[expert]], scale = max|v| / 127, q = v / scale.
template <typename T>
__global__ void __launch_bounds__(128) routing_quant_kernel(const RoutingParams p)
{
    __shared__ float red[4];
    const int pos = blockIdx.x;
    if (pos >= *p.total) return;
    const int j = p.sorted_row[pos];
    const T *row = reinterpret_cast<const T *>(p.x) + (size_t)(j / p.k) * p.h;
    const float *smooth = p.scale ? p.scale + (size_t)(__ldg(p.expert_idx + j) - p.e_start) * p.h : nullptr;
    float amax = 0.0f;
    for (int c = threadIdx.x; c < p.h; c += blockDim.x) {
        float v = to_f32(row[c]);
        if (smooth) v = __fmul_rn(v, __ldg(smooth + c));
        amax = fmaxf(amax, fabsf(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float scale = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) p.expanded_scale[pos] = scale;
    int8_t *out = reinterpret_cast<int8_t *>(p.expanded_x) + (size_t)pos * p.h;
    if (p.vec_ok) {  // four outputs per store; the second read of the row comes from L1 / L2
        for (int c = threadIdx.x * 4; c < p.h; c += blockDim.x * 4) {
            char4 q;
            float v0 = to_f32(row[c]), v1 = to_f32(row[c + 1]), v2 = to_f32(row[c + 2]), v3 = to_f32(row[c + 3]);
            if (smooth) {
                const float4 s = __ldg(reinterpret_cast<const float4 *>(smooth + c));
                v0 = __fmul_rn(v0, s.x); v1 = __fmul_rn(v1, s.y); v2 = __fmul_rn(v2, s.z); v3 = __fmul_rn(v3, s.w);
            }
            q.x = quant_trunc_round(v0, scale); q.y = quant_trunc_round(v1, scale);
            q.z = quant_trunc_round(v2, scale); q.w = quant_trunc_round(v3, scale);
            *reinterpret_cast<char4 *>(out + c) = q;
        }
    } else {
        for (int c = threadIdx.x; c < p.h; c += blockDim.x) {
            float v = to_f32(row[c]);
            if (smooth) v = __fmul_rn(v, __ldg(smooth + c));
            out[c] = quant_trunc_round(v, scale);
        }
    }
}

// The same value as quant_trunc_round in five instructions after the division, for the register-tiled kernel.  With
// |v / scale| <= 127 (scale is the row maximum over 127): fp16 towards zero keeps 11 significant bits, i.e. clears the low
// 13 mantissa bits of the fp32 quotient (below 2^-14, where fp16 is subnormal, both forms end as 0); adding 0.5 with the
// quotient's sign is exact and truncation then rounds ties away from zero; 0 / 0 stays NaN and converts to 0.
// `rcp` is the correctly rounded reciprocal of `scale` (or 0 to ask for the plain division): the quotient is then formed
// with fused multiply-adds, q0 = v * rcp, twice q = q + (v - q * scale) * rcp.  After the first correction q is a faithful
// rounding of v / scale, and with an exact residual and a correctly rounded reciprocal the second correction yields the
// correctly rounded quotient (Markstein's division theorem), i.e. the value __fdiv_rn returns, in five instructions.
__device__ __forceinline__ float exact_div(float v, float scale, float rcp)
{
    if (rcp == 0.0f) return __fdiv_rn(v, scale);
    float q = __fmul_rn(v, rcp);
    q = __fmaf_rn(__fmaf_rn(-q, scale, v), rcp, q);
    q = __fmaf_rn(__fmaf_rn(-q, scale, v), rcp, q);
    return q;
}

// 1 / scale for exact_div, or 0 where the shortcut is not safe (zero, denormal-range or huge scales).
__device__ __forceinline__ float exact_div_rcp(float scale)
{
    return (scale > 1e-30f && scale < 1e30f) ? __frcp_rn(scale) : 0.0f;
}

__device__ __forceinline__ int quant_fast(float v, float scale, float rcp)
{
    const uint32_t b = __float_as_uint(exact_div(v, scale, rcp)) & 0xffffe000u;
    const float r = __fadd_rn(__uint_as_float(b), __uint_as_float(0x3f000000u | (b & 0x80000000u)));
    return max(-128, min(127, __float2int_rz(r)));  // the clamp only matters for rows of denormals, whose scale underflows
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d)
{
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

template <int THREADS>
__device__ __forceinline__ float block_max(float v, float *red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();  // red may still be read from the previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[0];
#pragma unroll
    for (int i = 1; i < THREADS / 32; ++i) m = fmaxf(m, red[i]);
    return m;
}

template <typename T>
__device__ __forceinline__ void unpack16(const uint4 &u, float *f);
template <>
__device__ __forceinline__ void unpack16<float>(const uint4 &u, float *f)
{
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4 &u, float *f)
{
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <>
__device__ __forceinline__ void unpack16<__half>(const uint4 &u, float *f)
{
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

// The fast form of the quantising gather: one CTA per TOKEN.  The row is read once, 16 bytes per thread and step, and
// stays in registers; without a smooth scale it is quantised once and the int8 row is stored at the output row of each
// of the token's k pairs; with one, every pair is scaled, reduced and quantised from the registers.  DRAM traffic is the
// algorithmic minimum: x once, every output row once.  Needs h a multiple of the 16-byte vector, h <= THREADS * NCH * VEC
// and 16-byte aligned pointers; other shapes take routing_quant_kernel.  MINB CTAs per SM: the 16-bit inputs run with 4
// (64 registers): 66 instead of 73 us per call on 4096 x 7168 bf16 tokens, because a CTA is a chain of load, block
// reduction and stores, and only other CTAs fill the gaps.
template <typename T, int NCH, int THREADS, int MINB = 3>
__global__ void __launch_bounds__(THREADS, MINB) routing_quant_token_kernel(const RoutingParams p)
{
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int G = 16 / VEC;  // 16-byte loads that make one 16-byte store of int8: a thread owns G adjacent ones
    static_assert(NCH % G == 0, "whole stores per thread");
    __shared__ float red[THREADS / 32];
    const int token = blockIdx.x;
    const int chunks = p.h / VEC;
    const uint4 *row = reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(p.x) + (size_t)token * p.h);
    float v[NCH][VEC];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = (threadIdx.x + (i / G) * THREADS) * G + (i % G);
        if (c < chunks) {
            unpack16<T>(__ldg(row + c), v[i]);
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[i][e] = 0.0f;
        }
    }
    const bool smooth = p.scale != nullptr;
    float scale = 0.0f;
    uint32_t w[NCH][VEC / 4];  // the quantised row, four int8 per word
    if (!smooth) {             // one quantisation serves all k pairs of the token
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < NCH; ++i)
#pragma unroll
            for (int e = 0; e < VEC; ++e) amax = fmaxf(amax, fabsf(v[i][e]));
        scale = __fdiv_rn(block_max<THREADS>(amax, red), 127.0f);
        const float rcp = exact_div_rcp(scale);
#pragma unroll
        for (int i = 0; i < NCH; ++i)
#pragma unroll
            for (int e4 = 0; e4 < VEC; e4 += 4)
                w[i][e4 / 4] = pack4(quant_fast(v[i][e4], scale, rcp), quant_fast(v[i][e4 + 1], scale, rcp),
                                     quant_fast(v[i][e4 + 2], scale, rcp), quant_fast(v[i][e4 + 3], scale, rcp));
    }
    pdl_wait();  // the row positions are complete
    for (int s = 0; s < p.k; ++s) {
        const long long j = (long long)token * p.k + s;
        const int pos = p.pair_pos[j];
        if (pos < 0) continue;  // uniform over the CTA
        if (smooth) {
            const float *sm = p.scale + (size_t)(__ldg(p.expert_idx + j) - p.e_start) * p.h;
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int c = (threadIdx.x + (i / G) * THREADS) * G + (i % G);
                if (c < chunks) {
#pragma unroll
                    for (int e4 = 0; e4 < VEC; e4 += 4) {
                        const float4 m = __ldg(reinterpret_cast<const float4 *>(sm + (size_t)c * VEC + e4));
                        amax = fmaxf(fmaxf(amax, fabsf(__fmul_rn(v[i][e4], m.x))), fabsf(__fmul_rn(v[i][e4 + 1], m.y)));
                        amax = fmaxf(fmaxf(amax, fabsf(__fmul_rn(v[i][e4 + 2], m.z))), fabsf(__fmul_rn(v[i][e4 + 3], m.w)));
                    }
                }
            }
            scale = __fdiv_rn(block_max<THREADS>(amax, red), 127.0f);
            const float rcp = exact_div_rcp(scale);
#pragma unroll
            for (int i = 0; i < NCH; ++i) {  // the products are formed again: keeping them would cost 64 registers
                const int c = (threadIdx.x + (i / G) * THREADS) * G + (i % G);
                if (c < chunks) {
#pragma unroll
                    for (int e4 = 0; e4 < VEC; e4 += 4) {
                        const float4 m = __ldg(reinterpret_cast<const float4 *>(sm + (size_t)c * VEC + e4));
                        w[i][e4 / 4] = pack4(quant_fast(__fmul_rn(v[i][e4], m.x), scale, rcp), quant_fast(__fmul_rn(v[i][e4 + 1], m.y), scale, rcp),
                                             quant_fast(__fmul_rn(v[i][e4 + 2], m.z), scale, rcp), quant_fast(__fmul_rn(v[i][e4 + 3], m.w), scale, rcp));
                    }
                }
            }
        }
        if (threadIdx.x == 0) p.expanded_scale[pos] = scale;
        int8_t *out = reinterpret_cast<int8_t *>(p.expanded_x) + (size_t)pos * p.h;
#pragma unroll
        for (int i = 0; i < NCH; i += G) {
            const int c = (threadIdx.x + (i / G) * THREADS) * G;
            if (c < chunks) {
                uint4 o;
                if (VEC == 8) o = make_uint4(w[i][0], w[i][VEC / 4 - 1], w[i + G - 1][0], w[i + G - 1][VEC / 4 - 1]);
                else o = make_uint4(w[i][0], w[i + 1 < NCH ? i + 1 : i][0], w[i + 2 < NCH ? i + 2 : i][0], w[i + G - 1][0]);
                *reinterpret_cast<uint4 *>(out + (size_t)c * VEC) = o;
            }
        }
    }
}

// One CTA per token: the row is read once, 16 bytes per thread and step, and stored at the output row of each pair.
__global__ void __launch_bounds__(128) routing_copy_token_kernel(const RoutingParams p, int row_bytes)
{
    const int token = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(p.x) + (size_t)token * row_bytes);
    const int chunks = row_bytes / 16;
    for (int c0 = 0; c0 < chunks; c0 += 128 * 4) {
        uint4 buf[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + i * 128 + threadIdx.x;
            if (c < chunks) buf[i] = __ldg(src + c);
        }
        for (int s = 0; s < p.k; ++s) {
            const int pos = p.pair_pos[(long long)token * p.k + s];
            if (pos < 0) continue;
            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<char *>(p.expanded_x) + (size_t)pos * row_bytes);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = c0 + i * 128 + threadIdx.x;
                if (c < chunks) dst[c] = buf[i];
            }
        }
    }
    if (p.scale && p.expanded_scale && threadIdx.x < p.k) {
        const int pos = p.pair_pos[(long long)token * p.k + threadIdx.x];
        if (pos >= 0) p.expanded_scale[pos] = __ldg(p.scale + token);
    }
}

// One CTA per output row: plain copy of the token row (any element size), and of the token's scale if one is given.
__global__ void __launch_bounds__(128) routing_copy_kernel(const RoutingParams p, int elem_bytes)
{
    const int pos = blockIdx.x;
    if (pos >= *p.total) return;
    const int j = p.sorted_row[pos];
    const size_t row_bytes = (size_t)p.h * elem_bytes;
    const char *src = reinterpret_cast<const char *>(p.x) + (size_t)(j / p.k) * row_bytes;
    char *dst = reinterpret_cast<char *>(p.expanded_x) + (size_t)pos * row_bytes;
    if ((row_bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.expanded_x)) & 15) == 0) {
        for (size_t c = threadIdx.x * 16; c < row_bytes; c += blockDim.x * 16)
            *reinterpret_cast<uint4 *>(dst + c) = __ldg(reinterpret_cast<const uint4 *>(src + c));
    } else {
        for (size_t c = threadIdx.x; c < row_bytes; c += blockDim.x) dst[c] = src[c];
    }
    if (p.scale && p.expanded_scale && threadIdx.x == 0) p.expanded_scale[pos] = __ldg(p.scale + j / p.k);
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

size_t init_routing_workspace_bytes(const InitRoutingProblem &r)
{
    const long long pairs = r.n * r.k;
    const long long nb = (pairs + kPairsPerBlock - 1) / kPairsPerBlock;
    const long long range = r.expert_end - r.expert_start;
    return 256 + 2 * align256((size_t)nb * range * 4) + align256((size_t)range * 4) + 2 * align256((size_t)pairs * 4);
}

cudaError_t init_routing_launch(const InitRoutingProblem &r, void *workspace, size_t workspace_bytes, cudaStream_t stream)
{
    const long long pairs = r.n * r.k;
    if (pairs <= 0) return cudaSuccess;
    if (workspace_bytes < init_routing_workspace_bytes(r) || !workspace) return cudaErrorInvalidValue;
    const long long nb = (pairs + kPairsPerBlock - 1) / kPairsPerBlock;
    const int range = (int)(r.expert_end - r.expert_start);
    if (pairs > 0x7fffffffll || nb > 0x7fffffffll || range <= 0 || (size_t)range * 4 > 48 * 1024) return cudaErrorInvalidValue;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    RoutingParams p;
    p.x = r.x; p.x_dtype = r.x_dtype; p.expert_idx = r.expert_idx; p.scale = r.scale;
    p.pairs = pairs; p.k = (int)r.k; p.h = (int)r.h;
    p.e_start = (int)r.expert_start; p.range = range; p.expert_num = (int)r.expert_num;
    p.quant = r.quant; p.row_idx_type = r.row_idx_type; p.count_type = r.count_type;
    p.vec_ok = (r.h % 4 == 0) && ((reinterpret_cast<uintptr_t>(r.scale) | reinterpret_cast<uintptr_t>(r.expanded_x)) & 15) == 0;
    p.expanded_x = r.expanded_x; p.expanded_row_idx = r.expanded_row_idx; p.counts_out = r.counts_out;
    p.expanded_scale = r.expanded_scale;
    p.total = reinterpret_cast<int *>(ws);
    size_t off = 256;
    p.block_hist = reinterpret_cast<int *>(ws + off); off += align256((size_t)nb * range * 4);
    p.block_off = reinterpret_cast<int *>(ws + off); off += align256((size_t)nb * range * 4);
    p.expert_first = reinterpret_cast<int *>(ws + off); off += align256((size_t)range * 4);
    p.sorted_row = reinterpret_cast<int *>(ws + off); off += align256((size_t)pairs * 4);
    p.pair_pos = reinterpret_cast<int *>(ws + off);
    p.nb = (int)nb;
    const size_t smem = (size_t)range * 4;
    // GMM_B200_PDL=0 turns the overlap of the chain's kernels off (plain stream order)
    const char *pdl_env = getenv("GMM_B200_PDL");
    const bool overlap = !(pdl_env && pdl_env[0] == '0');
    routing_count_kernel<<<(unsigned)nb, kPairsPerBlock, smem, stream>>>(p);
    if (range <= kWarpTableRange && (long long)nb * range <= kFoldTable) {
        const cudaError_t e = launch_pdl(routing_scatter_kernel<true, true>, (unsigned)nb, kPairsPerBlock, smem * (kPairsPerBlock / 32), stream, overlap, p);
        if (e != cudaSuccess) return e;
    } else {
        routing_scan_kernel<<<(unsigned)((range + 31) / 32), 1024, 0, stream>>>(p);
        if (range <= kWarpTableRange) routing_scatter_kernel<true><<<(unsigned)nb, kPairsPerBlock, smem * (kPairsPerBlock / 32), stream>>>(p);
        else routing_scatter_kernel<false><<<(unsigned)nb, kPairsPerBlock, smem, stream>>>(p);
    }
    const int eb = r.x_dtype == kF32 ? 4 : (r.x_dtype == kI8 ? 1 : 2);
    const bool aligned = ((reinterpret_cast<uintptr_t>(r.x) | reinterpret_cast<uintptr_t>(r.expanded_x) | reinterpret_cast<uintptr_t>(r.scale)) & 15) == 0;
    cudaError_t launch_err = cudaSuccess;
    if (r.quant) {
        // token-major kernels hold 32 values per thread (256 threads): h <= 8192, and h a multiple of 16 for the 16-byte stores
        const bool fast = aligned && r.h % 16 == 0 && r.h <= 8192 && r.n <= 0x7fffffffll;
        if (r.x_dtype == kF32) {
            if (fast) launch_err = launch_pdl(routing_quant_token_kernel<float, 8, 256>, (unsigned)r.n, 256, 0, stream, overlap, p);
            else routing_quant_kernel<float><<<(unsigned)pairs, 128, 0, stream>>>(p);
        } else if (r.x_dtype == kF16) {
            if (fast) launch_err = launch_pdl(routing_quant_token_kernel<__half, 4, 256, 4>, (unsigned)r.n, 256, 0, stream, overlap, p);
            else routing_quant_kernel<__half><<<(unsigned)pairs, 128, 0, stream>>>(p);
        } else if (r.x_dtype == kBF16) {
            if (fast) launch_err = launch_pdl(routing_quant_token_kernel<__nv_bfloat16, 4, 256, 4>, (unsigned)r.n, 256, 0, stream, overlap, p);
            else routing_quant_kernel<__nv_bfloat16><<<(unsigned)pairs, 128, 0, stream>>>(p);
        } else {
            return cudaErrorInvalidValue;
        }
    } else {
        const long long row_bytes = r.h * eb;
        if (aligned && row_bytes % 16 == 0 && row_bytes <= 0x7fffffffll && r.k <= 128)
            routing_copy_token_kernel<<<(unsigned)r.n, 128, 0, stream>>>(p, (int)row_bytes);
        else
            routing_copy_kernel<<<(unsigned)pairs, 128, 0, stream>>>(p, eb);
    }
    if (launch_err != cudaSuccess) return launch_err;
    return cudaGetLastError();
}

}  // namespace gmm
