// Grouped int8 GEMM for sm_100a: TMA-staged tiles -> tcgen05.mma kind::i8 -> TMEM int32 accumulators ->
// warp-specialised fused epilogue.  One persistent CTA per SM walks a tile list that every CTA derives
// from group_list on the device (empty experts produce no tiles).
//
// Replaces, for NVIDIA B200, the reference's AscendC kernels
//   gmm/grouped_matmul/op_kernel/grouped_matmul.h:250-283            (GMMProcess::Process, the block scheduler)
//   gmm/grouped_matmul/op_kernel/grouped_matmul_quant_mixcore.h:175-315 (int8 matmul + dequant epilogue)
//   gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant.h:231-262, 367-474 (matmul, dequant, SwiGLU)
// and the host tiling that feeds them (op_host/op_tiling/grouped_matmul_tiling.cpp:727-763).
//
// Tile: 128 rows x 256 accumulator columns, K consumed 128 bytes per pipeline stage (4 MMAs of K=32).
//   grouped_matmul       : the 256 columns are 256 consecutive output columns.
//   swiglu_quant         : columns [0,128) come from weight columns n0.. (activated half), columns [128,256)
//                          from N/2+n0.. (linear half), so SwiGLU is tile-local and a tile yields 128 outputs.
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2-9 = epilogue.
// Every wait on an mbarrier is bounded; on expiry the CTA records a status word, all roles leave their loops,
// outstanding copies are drained with a second bounded wait, TMEM is released and the kernel returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gmm_common.h"

namespace gmm {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int STAGES = 4;
constexpr int UMMA_K = 32;
constexpr int A_STAGE = BM * BK;
constexpr int B_STAGE = BN * BK;
constexpr int B_HALF = B_STAGE / 2;
constexpr int STAGE_BYTES = A_STAGE + B_STAGE;
constexpr int MAX_GROUPS = 1024;
constexpr int EPI_WARPS = 8;                 // two warps per TMEM lane quarter, each takes half of the columns
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_LIMIT_CYCLES = 1ll << 31;   // about a second
constexpr long long DRAIN_LIMIT_CYCLES = 1ll << 24;  // a few milliseconds

struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int total_tiles;
    int pad;
    int row_start[MAX_GROUPS];
    int rows[MAX_GROUPS];
    int tile_start[MAX_GROUPS + 1];
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + sizeof(Shared);

struct KParams {
    const int64_t *group_list;
    int gl_len, gl_type;
    int M, K, N;
    int half_n;        // N/2 (swiglu)
    int n_tiles;       // tiles along N per row block
    int num_k_blocks;  // ceil(K / BK)
    const void *w_scale;
    int w_scale_dtype;
    const float *x_scale;
    const void *bias;
    int bias_dtype;
    int act_type;
    void *out;            // y (bf16 / int32) or the fp32 SwiGLU staging [M, N/2]
    unsigned *amax_bits;  // [M] row max of |S| as float bits, top bit set once written (swiglu)
    int *status;
};

// ---------------------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out or another role already gave up.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, Shared *sh, int *status, int who,
                                            long long limit)
{
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0u) {
            if (*(volatile int *)&sh->abort_flag) return false;
            if (clock64() - t0 > limit) {
                *(volatile int *)&sh->abort_flag = 1;
                if (atomicCAS(status, kStatusOk, kStatusWaitTimeout) == kStatusOk) {
                    status[1] = (int)blockIdx.x;
                    status[2] = who;
                    status[3] = (int)parity;
                }
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, Shared *sh, int *status, int who)
{
    const uint32_t a = smem_u32(bar);
    if (mbar_try_wait(a, parity)) return true;
    return mbar_wait_slow(a, parity, sh, status, who, WAIT_LIMIT_CYCLES);
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], int8 x int8 -> int32, issued by one thread.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit values: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
//   K-major operand : rows of 128 bytes, 8-row groups 1024 bytes apart (SBO); LBO unused.
//   MN-major operand: 128-byte runs along M/N; the next 8 K-rows are SBO bytes on, the next 128 M/N LBO bytes on.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::i8: D = S32 (2 at bit 4), A = B = signed 8-bit (1 at bits 7 and 10),
// A K-major, B major per flag (bit 16), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(bool b_mn_major)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------------------
// Tile schedule, rebuilt by every CTA from group_list (<= 1024 entries)
// ---------------------------------------------------------------------------------------------------------

// Row ranges follow GetSplitValueFromGroupList (gmm/grouped_matmul/op_kernel/grouped_matmul_utils.h:243-257):
// type 0 = running total, type 1 = count, values narrowed to int32; groups with no rows are skipped
// (grouped_matmul.h:263).  Ranges are clipped to [0, M] so a malformed list cannot address other memory.
__device__ void build_schedule(Shared *sh, const KParams &p)
{
    const int tid = threadIdx.x, L = p.gl_len;
    for (int g = tid; g < L; g += NUM_THREADS) {
        const int v = (int)p.group_list[g];
        int start = 0, rows = v;
        if (p.gl_type == 0) {
            const int prev = g ? (int)p.group_list[g - 1] : 0;
            start = prev;
            rows = v - prev;
        }
        sh->row_start[g] = start;
        sh->rows[g] = rows;
    }
    __syncthreads();
    if (tid < 32) {
        const int lane = tid;
        const int chunk = (L + 31) / 32;
        const int lo = min(lane * chunk, L), hi = min(lo + chunk, L);
        if (p.gl_type != 0) {
            int s = 0;
            for (int g = lo; g < hi; ++g) s += max(sh->rows[g], 0);
            int incl = s;
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            int run = incl - s;
            for (int g = lo; g < hi; ++g) {
                sh->row_start[g] = run;
                run += max(sh->rows[g], 0);
            }
        }
        int tsum = 0;
        for (int g = lo; g < hi; ++g) {
            long long start = sh->row_start[g], rows = sh->rows[g];
            if (rows < 0) rows = 0;
            if (start < 0) { rows += start; start = 0; if (rows < 0) rows = 0; }
            if (start > p.M) { start = p.M; rows = 0; }
            if (start + rows > p.M) rows = p.M - start;
            sh->row_start[g] = (int)start;
            sh->rows[g] = (int)rows;
            tsum += (int)((rows + BM - 1) / BM) * p.n_tiles;
        }
        int incl = tsum;
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        int run = incl - tsum;
        for (int g = lo; g < hi; ++g) {
            sh->tile_start[g] = run;
            run += ((sh->rows[g] + BM - 1) / BM) * p.n_tiles;
        }
        if (lane == 31) {
            sh->tile_start[L] = incl;
            sh->total_tiles = incl;
        }
    }
    __syncthreads();
}

struct Tile {
    int g, row0, rows, n_idx;
};

__device__ __forceinline__ Tile decode_tile(const Shared *sh, int t, int n_tiles, int L)
{
    int lo = 0, hi = L;  // largest g in [0, L) with tile_start[g] <= t
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (sh->tile_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int local = t - sh->tile_start[lo];
    const int mb = local / n_tiles;
    Tile tl;
    tl.g = lo;
    tl.n_idx = local - mb * n_tiles;
    tl.row0 = sh->row_start[lo] + mb * BM;
    tl.rows = min(BM, sh->rows[lo] - mb * BM);
    return tl;
}

// ---------------------------------------------------------------------------------------------------------
// Epilogue helpers
// ---------------------------------------------------------------------------------------------------------

__device__ __forceinline__ void load_scales8(const void *p, int dtype, size_t i, float (&s)[8])
{
    if (dtype == kF32) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i) + 1);
        s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w; s[4] = b.x; s[5] = b.y; s[6] = b.z; s[7] = b.w;
    } else {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p) + i));
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (dtype == kBF16) {
                s[2 * j] = __uint_as_float(w[j] << 16);
                s[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            } else {
                const __half2 h = *reinterpret_cast<const __half2 *>(&w[j]);
                s[2 * j] = __low2float(h);
                s[2 * j + 1] = __high2float(h);
            }
        }
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    const __nv_bfloat16 a = __float2bfloat16_rn(lo), b = __float2bfloat16_rn(hi);
    return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

// ---------------------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------------------

template <int MODE, bool B_MN_MAJOR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gmm_w8a8_sm100_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const KParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + STAGES * A_STAGE;
    Shared *sh = reinterpret_cast<Shared *>(smem + STAGES * STAGE_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh->acc_full[b], 1);
            mbar_init(&sh->acc_empty[b], 32 * EPI_WARPS);
        }
        sh->abort_flag = 0;
        sh->total_tiles = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&map_x);
        prefetch_map(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, TMEM_COLS);
        tc_fence_before();
    }
    build_schedule(sh, p);  // ends with __syncthreads()
    tc_fence_after();

    const int total_tiles = sh->total_tiles;
    const uint32_t tmem_base = sh->tmem_base;
    const int L = p.gl_len;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const Tile tl = decode_tile(sh, t, p.n_tiles, L);
                int n0, n1;
                if (MODE == kModeSwigluQuant) { n0 = tl.n_idx * (BN / 2); n1 = p.half_n + n0; }
                else { n0 = tl.n_idx * BN; n1 = n0 + BN / 2; }
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    if (!mbar_wait(&sh->empty[stage], phase ^ 1u, sh, p.status, 100 + stage)) { ok = false; break; }
                    mbar_arrive_expect_tx(&sh->full[stage], STAGE_BYTES);
                    tma_load_2d(smem_a + stage * A_STAGE, &map_x, kb * BK, tl.row0, &sh->full[stage]);
                    uint8_t *bdst = smem_b + stage * B_STAGE;
                    if (B_MN_MAJOR) {  // weight [E, K, N]: map dims {N, K, E}
                        tma_load_3d(bdst, &map_w, n0, kb * BK, tl.g, &sh->full[stage]);
                        tma_load_3d(bdst + B_HALF, &map_w, n1, kb * BK, tl.g, &sh->full[stage]);
                    } else {           // weight [E, N, K]: map dims {K, N, E}
                        tma_load_3d(bdst, &map_w, kb * BK, n0, tl.g, &sh->full[stage]);
                        tma_load_3d(bdst + B_HALF, &map_w, kb * BK, n1, tl.g, &sh->full[stage]);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok || *(volatile int *)&sh->abort_flag) {
                // Drain: give the copies already issued a bounded chance to land before the CTA leaves.
                const int n = (int)(issued < STAGES ? issued : STAGES);
                int s = stage;
                uint32_t ph = phase;
                for (int i = 0; i < n; ++i) {
                    if (--s < 0) { s = STAGES - 1; ph ^= 1u; }
                    const uint32_t a = smem_u32(&sh->full[s]);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(a, ph) && clock64() - t0 < DRAIN_LIMIT_CYCLES) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(B_MN_MAJOR);
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(&sh->acc_empty[buf], acc_phase ^ 1u, sh, p.status, 200 + buf)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    if (!mbar_wait(&sh->full[stage], phase, sh, p.status, 300 + stage)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + stage * A_STAGE);
                    const uint32_t b_addr = smem_u32(smem_b + stage * B_STAGE);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        const uint64_t a_desc = make_smem_desc(a_addr + j * UMMA_K, 16, 1024);
                        const uint64_t b_desc = B_MN_MAJOR ? make_smem_desc(b_addr + j * UMMA_K * 128, B_HALF, 1024)
                                                           : make_smem_desc(b_addr + j * UMMA_K, 16, 1024);
                        umma_i8(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    umma_commit(&sh->empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&sh->acc_full[buf]);
                buf ^= 1;
                if (buf == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------ epilogue: warp -> (TMEM lane quarter, column half) ------------------------------
        const int quarter = warp & 3;
        const int chalf = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
        int buf = 0;
        uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
            const Tile tl = decode_tile(sh, t, p.n_tiles, L);
            const bool valid = r < tl.rows;
            const bool warp_has_rows = quarter * 32 < tl.rows;
            const int grow = tl.row0 + r;
            const float xs = (valid && p.x_scale) ? __ldg(p.x_scale + grow) : 1.0f;
            if (!mbar_wait(&sh->acc_full[buf], acc_phase, sh, p.status, 400 + buf)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * BN;

            if (warp_has_rows) {
                if (MODE == kModeSwigluQuant) {
                    const int n0 = tl.n_idx * (BN / 2);
                    float amax = 0.0f;
                    float *srow = reinterpret_cast<float *>(p.out) + (size_t)grow * p.half_n;
                    const size_t sbase = (size_t)tl.g * p.N;
#pragma unroll 1
                    for (int c = chalf * 2; c < chalf * 2 + 2; ++c) {
                        uint32_t va[32], vb[32];
                        tmem_ld32(taddr + c * 32, va);
                        tmem_ld32(taddr + BN / 2 + c * 32, vb);
                        tmem_ld_wait();
#pragma unroll
                        for (int j8 = 0; j8 < 4; ++j8) {
                            const int col = n0 + c * 32 + j8 * 8;
                            if (col < p.half_n) {
                                float sa[8], sb[8], o[8];
                                load_scales8(p.w_scale, p.w_scale_dtype, sbase + col, sa);
                                load_scales8(p.w_scale, p.w_scale_dtype, sbase + p.half_n + col, sb);
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    // (acc * x_scale) * w_scale, then S = gate * (act / (1 + exp(-act)))
                                    float a = __fmul_rn(__fmul_rn(__int2float_rn((int)va[j8 * 8 + j]), xs), sa[j]);
                                    float b = __fmul_rn(__fmul_rn(__int2float_rn((int)vb[j8 * 8 + j]), xs), sb[j]);
                                    const float den = __fadd_rn(1.0f, expf(-a));
                                    const float sw = __fdiv_rn(a, den);
                                    const float s = __fmul_rn(b, sw);
                                    o[j] = s;
                                    amax = fmaxf(amax, fabsf(s));
                                }
                                if (valid) {
                                    float4 *dst = reinterpret_cast<float4 *>(srow + col);
                                    dst[0] = make_float4(o[0], o[1], o[2], o[3]);
                                    dst[1] = make_float4(o[4], o[5], o[6], o[7]);
                                }
                            }
                        }
                    }
                    if (valid) atomicMax(p.amax_bits + grow, __float_as_uint(amax) | 0x80000000u);  // top bit: row written
                } else {
                    const int n0 = tl.n_idx * BN;
                    const size_t sbase = (size_t)tl.g * p.N;
#pragma unroll 1
                    for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
                        if (n0 + c * 32 >= p.N) break;
                        uint32_t v[32];
                        tmem_ld32(taddr + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j8 = 0; j8 < 4; ++j8) {
                            const int col = n0 + c * 32 + j8 * 8;
                            if (col < p.N) {
                                int acc[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) acc[j] = (int)v[j8 * 8 + j];
                                if (p.bias_dtype == kI32) {
                                    const int4 b0 = __ldg(reinterpret_cast<const int4 *>(reinterpret_cast<const int *>(p.bias) + sbase + col));
                                    const int4 b1 = __ldg(reinterpret_cast<const int4 *>(reinterpret_cast<const int *>(p.bias) + sbase + col) + 1);
                                    acc[0] += b0.x; acc[1] += b0.y; acc[2] += b0.z; acc[3] += b0.w;
                                    acc[4] += b1.x; acc[5] += b1.y; acc[6] += b1.z; acc[7] += b1.w;
                                }
                                if (MODE == kModeInt32) {
                                    if (valid) {
                                        int4 *dst = reinterpret_cast<int4 *>(reinterpret_cast<int *>(p.out) + (size_t)grow * p.N + col);
                                        dst[0] = make_int4(acc[0], acc[1], acc[2], acc[3]);
                                        dst[1] = make_int4(acc[4], acc[5], acc[6], acc[7]);
                                    }
                                } else {
                                    float sc[8], o[8];
                                    load_scales8(p.w_scale, p.w_scale_dtype, sbase + col, sc);
                                    float bf[8];
                                    if (p.bias_dtype == kBF16) load_scales8(p.bias, kBF16, sbase + col, bf);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        // (acc * w_scale) * x_scale, optional bf16 bias, optional relu, bf16 RNE
                                        float tv = __fmul_rn(__int2float_rn(acc[j]), sc[j]);
                                        if (p.x_scale) tv = __fmul_rn(tv, xs);
                                        if (p.bias_dtype == kBF16) tv = __fadd_rn(tv, bf[j]);
                                        if (p.act_type == 1) tv = tv > 0.0f ? tv : 0.0f;
                                        o[j] = tv;
                                    }
                                    if (valid) {
                                        uint4 pk;
                                        pk.x = pack_bf16x2(o[0], o[1]);
                                        pk.y = pack_bf16x2(o[2], o[3]);
                                        pk.z = pack_bf16x2(o[4], o[5]);
                                        pk.w = pack_bf16x2(o[6], o[7]);
                                        *reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(p.out) + (size_t)grow * p.N + col) = pk;
                                    }
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&sh->acc_empty[buf]);
            buf ^= 1;
            if (buf == 0) acc_phase ^= 1u;
        }
    }

    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

template <int MODE, bool B_MN>
cudaError_t launch_variant(const Plan &plan, const KParams &kp, cudaStream_t stream)
{
    auto kern = gmm_w8a8_sm100_kernel<MODE, B_MN>;
    // Once per device and instantiation; the attribute is idempotent, so a race only repeats the call.
    static unsigned long long done_mask = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!((done_mask >> (dev & 63)) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return e;
        done_mask |= 1ull << (dev & 63);
    }
    kern<<<plan.num_sms, NUM_THREADS, SMEM_BYTES, stream>>>(plan.map_x, plan.map_w, kp);
    return cudaGetLastError();
}

cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;

}  // namespace

void set_timing_events(cudaEvent_t start, cudaEvent_t stop)
{
    g_ev_start = start;
    g_ev_stop = stop;
}

// The tcgen05 path needs 16-byte aligned row pitches for TMA (K for x; N or K for the weight), 16-byte
// aligned base pointers and, for SwiGLU, a half width that keeps the second box aligned.
bool sm100_shape_ok(const Problem &p)
{
    if (p.K % 16 != 0 || p.N % 16 != 0) return false;
    if (p.mode == kModeSwigluQuant && p.N % 32 != 0) return false;
    if (p.gl_len > MAX_GROUPS || p.gl_len <= 0) return false;
    if (p.M <= 0 || p.M > 0x7fffffffll / 2 || p.K > 0x7fffffffll || p.N > 0x7fffffffll) return false;
    if ((reinterpret_cast<uintptr_t>(p.x) & 15) || (reinterpret_cast<uintptr_t>(p.w) & 15)) return false;
    if (reinterpret_cast<uintptr_t>(p.out0) & 15) return false;
    if (reinterpret_cast<uintptr_t>(p.w_scale) & 15) return false;
    if (p.bias && (reinterpret_cast<uintptr_t>(p.bias) & 15)) return false;
    return true;
}

cudaError_t sm100_encode_maps(const Problem &p, Plan &plan)
{
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    {
        cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
        cuuint64_t strides[1] = {(cuuint64_t)p.K};
        cuuint32_t box[2] = {BK, BM};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&plan.map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(p.x), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t inner = p.w_trans ? p.K : p.N, mid = p.w_trans ? p.N : p.K;
        cuuint64_t dims[3] = {inner, mid, (cuuint64_t)p.E};
        cuuint64_t strides[2] = {inner, inner * mid};
        cuuint32_t box[3] = {128, 128, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = enc(&plan.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t *>(p.w), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    plan.maps_ready = true;
    return cudaSuccess;
}

cudaError_t sm100_launch(const Problem &p, Plan &plan, void *workspace, cudaStream_t stream)
{
    if (!plan.maps_ready) {
        cudaError_t e = sm100_encode_maps(p, plan);
        if (e != cudaSuccess) return e;
    }
    if (plan.num_sms <= 0) plan.num_sms = device_sm_count();
    if (plan.num_sms <= 0) return cudaErrorNoDevice;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    KParams kp;
    kp.group_list = p.group_list;
    kp.gl_len = p.gl_len;
    kp.gl_type = p.gl_type;
    kp.M = (int)p.M;
    kp.K = (int)p.K;
    kp.N = (int)p.N;
    kp.half_n = (int)(p.N / 2);
    kp.n_tiles = p.mode == kModeSwigluQuant ? (int)((p.N / 2 + BN / 2 - 1) / (BN / 2)) : (int)((p.N + BN - 1) / BN);
    kp.num_k_blocks = (int)((p.K + BK - 1) / BK);
    kp.w_scale = p.w_scale;
    kp.w_scale_dtype = p.w_scale_dtype;
    kp.x_scale = p.x_scale;
    kp.bias = p.bias;
    kp.bias_dtype = p.bias ? p.bias_dtype : kNone;
    kp.act_type = p.act_type;
    kp.status = reinterpret_cast<int *>(ws + plan.off_status);
    kp.amax_bits = reinterpret_cast<unsigned *>(ws + plan.off_amax);
    kp.out = p.mode == kModeSwigluQuant ? static_cast<void *>(ws + plan.off_stage) : p.out0;

    cudaError_t e;
    const bool mn = !p.w_trans;
    if (g_ev_start) cudaEventRecord(g_ev_start, stream);
    if (p.mode == kModeSwigluQuant)
        e = mn ? launch_variant<kModeSwigluQuant, true>(plan, kp, stream) : launch_variant<kModeSwigluQuant, false>(plan, kp, stream);
    else if (p.mode == kModeInt32)
        e = mn ? launch_variant<kModeInt32, true>(plan, kp, stream) : launch_variant<kModeInt32, false>(plan, kp, stream);
    else
        e = mn ? launch_variant<kModeDequantBf16, true>(plan, kp, stream) : launch_variant<kModeDequantBf16, false>(plan, kp, stream);
    if (g_ev_stop) cudaEventRecord(g_ev_stop, stream);
    if (e != cudaSuccess) return e;
    if (p.mode == kModeSwigluQuant)
        e = quant_rows_launch(p, reinterpret_cast<const float *>(ws + plan.off_stage), kp.amax_bits, stream);
    return e;
}

}  // namespace gmm
