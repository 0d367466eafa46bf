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
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2-9 = epilogue; swiglu_quant
// adds warp 10, one lane of which keeps the books of the row blocks in global memory.
// CTA pairs (cluster of 2, tcgen05 cta_group::2) compute 256-row tiles when groups are long; each CTA then stages its own
// 128 rows of x and half of the weight columns.  Weight layouts: [E,K,N] (MN-major operand, 128-byte swizzle), the
// transposed view [E,N,K] (K-major) and FRACTAL_NZ [E,N/32,K/16,16,32] (MN-major, 32-byte swizzle, 5-D tensor map).
// Epilogue: the tile's per-column scales are staged in shared memory while the MMAs run; bf16 / fp16 results are
// transposed through shared memory so that stores cover whole 128-byte row segments (optionally scattered by a row
// index, also into other GPUs' buffers); the finalize-routing variant adds weighted fp32 rows into token rows with
// 16-byte vector reductions; SwiGLU values go to an fp32 staging buffer (transposed the same way) with a per-row atomic
// max, and a finished row block is requantised to int8 in row slices that the CTAs which worked on it claim from a
// counter - no CTA ever waits for another one (see publish_and_collect).
// What bounds the MMA loop is the shared-memory / L1 data path (TMA writes, operand reads of both CTAs of a pair, and
// every load, store and shuffle of the epilogue), not the tensor pipe and not the feed: memory instructions of the
// epilogue are kept wide and contiguous for that reason.  The producers pace themselves wave by wave so that the units
// which share x rows and weight boxes through L2 stay together (a bounded hint).
// Every wait on an mbarrier is bounded; on expiry the CTA records a status word, all roles leave their loops,
// outstanding copies are drained with a second bounded wait, TMEM is released and the kernel returns.
// -DGMM_TRACE builds in clock64 / globaltimer stamps of the roles of a few CTAs (a buffer address comes from the environment).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstddef>
#include <cstdlib>

#include "gmm_common.h"

namespace gmm {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int A_STAGE = BM * BK;        // 128 rows x 128 bytes of K
constexpr int B_BOX = 128 * BK;         // one weight box: 128 N-columns x 128 bytes of K
constexpr int PIPE_BYTES = 196608;      // shared memory given to the TMA ring
constexpr int MAX_STAGES = 6;

// CTAS = 1: one CTA computes a 128 x 256 tile; it stages A (16 KB) and both weight boxes (32 KB) per K block, 4 stages.
// CTAS = 2: a pair of CTAs (one cluster) computes a 256 x 256 tile with cta_group::2 MMAs; each CTA stages its own 128
//           rows of A and ONE weight box (its half of the 256 columns), so a K block costs 32 KB per SM and the ring
//           holds 6 stages.  The pair's even CTA issues the MMAs for both.
template <int CTAS>
struct Cfg {
    static constexpr int kBoxes = 2 / CTAS;                 // weight boxes staged per CTA and K block
    static constexpr int kStageBytes = A_STAGE + kBoxes * B_BOX;
    static constexpr int kStages = PIPE_BYTES / kStageBytes;
    static constexpr int kTileM = BM * CTAS;
    static constexpr uint32_t kTxBytes = (uint32_t)kStageBytes * CTAS;  // bytes landing per stage, both CTAs together
};
static_assert(Cfg<1>::kStages == 4 && Cfg<2>::kStages == 6 && Cfg<2>::kStages <= MAX_STAGES, "stage arithmetic");
constexpr int MAX_GROUPS = 1024;
constexpr int EPI_WARPS = 8;                 // two warps per TMEM lane quarter, each takes half of the columns
// swiglu_quant only: one more warp, of which one lane keeps the books of the row blocks in global memory (arrivals, slice
// claims) beside the epilogue, so that none of its round trips to L2 delays the next tile.  It hands the epilogue warps
// lists of row ranges to requantise through a small ring.
constexpr int WK_DEPTH = 4;                  // work lists the publishing lane may be ahead of the epilogue warps
constexpr int BASE_THREADS = 64 + 32 * EPI_WARPS;
__host__ __device__ constexpr int num_threads(int mode) { return BASE_THREADS + (mode == kModeSwigluQuant ? 32 : 0); }
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_LIMIT_CYCLES = 1ll << 31;   // about a second
constexpr long long DRAIN_LIMIT_CYCLES = 1ll << 24;  // a few milliseconds
// Upper bound (ns) of the time a thread may stay suspended inside one mbarrier.try_wait before it polls again.  The board
// is power capped under these kernels, so waiting warps that poll less leave more of the budget to the clock: with 2 us
// instead of the default C3 runs 0.399 instead of 0.414 ms, C2 0.80-0.81 instead of 0.82-0.83 ms (same box, alternating).
constexpr uint32_t WAIT_SUSPEND_NS = 2000;

constexpr int EPI_THREADS = 32 * EPI_WARPS;
enum : int { kEpiPlain = 0, kEpiScatter = 1, kEpiGeneric = 2, kEpiCombine = 3 };
// Weight layouts: [E,K,N]; [E,N,K] (the transposed view); FRACTAL_NZ [E, N/32, K/16, 16, 32] (32-byte runs along N).
enum : int { kBRowMajor = 0, kBTransposed = 1, kBFractalNz = 2 };
constexpr int MAX_PENDING = 6;         // unsettled row blocks a CTA keeps track of before it hands its share over
constexpr int SCALE_BUFS = 3;          // an epilogue thread can run at most two tiles ahead of another one
constexpr int OUT_STAGE_BYTES = 2048;  // per epilogue warp: 32 rows x 64 bytes of packed bf16

struct Shared {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t scale_ready[SCALE_BUFS];  // all epilogue threads have stored their column's scale
    uint64_t wk_full[WK_DEPTH];        // a work list is written (swiglu_quant)
    uint64_t wk_empty[WK_DEPTH];       // every epilogue warp is done with it
    uint32_t tmem_base;
    int abort_flag;
    int total_tiles;
    int pad;
    long long wait_limit;              // bound of every wait, in cycles
    // swiglu_quant: how many epilogue threads have stored (and fenced) their part of how many tiles; the row blocks this
    // CTA contributed to and has not yet settled (publishing lane only); a ring of work lists: the row ranges to requantise
    // (written by that lane, read by the epilogue warps after wk_full)
    unsigned stored_count;
    int pend_n;
    int pend_rb[MAX_PENDING], pend_row0[MAX_PENDING], pend_rows[MAX_PENDING];
    int n_work[WK_DEPTH];
    int work_begin[WK_DEPTH][MAX_PENDING + 1], work_end[WK_DEPTH][MAX_PENDING + 1];
    int row_start[MAX_GROUPS];
    int rows[MAX_GROUPS];
    int tile_start[MAX_GROUPS + 1];
    alignas(16) float scales[SCALE_BUFS][BN];  // dequant scale of every accumulator column of the tile (read as float4)
    alignas(16) uint8_t out_stage[EPI_WARPS][OUT_STAGE_BYTES];
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)PIPE_BYTES + sizeof(Shared);
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
static_assert(offsetof(Shared, scales) % 16 == 0 && offsetof(Shared, out_stage) % 16 == 0, "vector accesses need 16-byte alignment");

// Debug build only (-DGMM_TRACE): clock64 stamps of the roles of a few CTAs, written to a buffer whose address comes from
// the environment; layout [cta < 4][role < 4][tile < 64][slot < 8].
#ifdef GMM_TRACE
#define TRACE(role, tile, slot)                                                                                           \
    do {                                                                                                                  \
        if (p.trace && blockIdx.x < 4 && (tile) < 64) p.trace[(((int)blockIdx.x * 4 + (role)) * 64 + (tile)) * 8 + (slot)] = clock64(); \
    } while (0)
#define TRACE_ADD(role, tile, slot, v)                                                                                    \
    do {                                                                                                                  \
        if (p.trace && blockIdx.x < 4 && (tile) < 64) p.trace[(((int)blockIdx.x * 4 + (role)) * 64 + (tile)) * 8 + (slot)] += (v); \
    } while (0)
#define TRACE_GT(role, tile, slot)                                                                                        \
    do {                                                                                                                  \
        unsigned long long gt_;                                                                                           \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                                                           \
        if (p.trace && blockIdx.x < 4 && (tile) < 64) p.trace[(((int)blockIdx.x * 4 + (role)) * 64 + (tile)) * 8 + (slot)] = (long long)gt_; \
    } while (0)
#else
#define TRACE_GT(role, tile, slot) do {} while (0)
#define TRACE(role, tile, slot) do {} while (0)
#define TRACE_ADD(role, tile, slot, v) do {} while (0)
#endif

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
    int act_type, out_f16;
    void *out;            // y (bf16 / int32) or the fp32 SwiGLU staging [M, N/2]
    const long long *out_row_index;  // optional: result row r is written to row out_row_index[r] (bf16 / int32 modes)
    void *out_peers[8];              // bf16 mode with num_peers > 0: out_row_index = (gpu << 40) | row, base per gpu here
    int num_peers;
    // combine epilogue (grouped_matmul_finalize_routing): fp32 result rows added to / stored at row row_index[r] of out
    const float *logit;        // [M] routing weight per row, may be null
    const void *row_index;     // [M] int64 or int32
    int row_index_i32;
    int scatter_add;           // 1: atomic adds (shared-expert rows and logits given), 0: plain stores
    long long out_rows;        // rows of the fp32 result; indices outside [0, out_rows) are skipped
    unsigned *amax_bits;  // [M] row max of |S| as float bits (swiglu)
    int *rb_counter;      // per row block of a tile two words: arrivals + (hand-overs << 16), and the slice claim counter (swiglu)
    int rb_base;          // first counter of this launch (two launches share the array)
    int part;             // 0: all rows; 1: every group without its trailing rows if those are at most 128; 2: only those
    int8_t *q_out;        // int8 [M, N/2] (swiglu)
    float *q_scale_out;   // fp32 [M] (swiglu)
    int *status;
    long long wait_limit;   // cycles a wait may last before the CTA gives up and records kStatusWaitTimeout
    int skip_k_blocks;      // test only: K blocks the producer leaves out of its last tile (drives the abort path)
    int *wave_cnt;          // optional: per wave (round of the static tile schedule) the units that have started it
    int pace_cycles;        // how long a producer waits for the other units to have started the previous wave
#ifdef GMM_TRACE
    long long *trace;
#endif
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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(WAIT_SUSPEND_NS)
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
    return mbar_wait_slow(a, parity, sh, status, who, sh->wait_limit);
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
__device__ __forceinline__ void tma_load_5d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar))
        : "memory");
}
// Pair (cta_group::2) forms: the copy lands in the executing CTA's shared memory, the byte count is credited to the
// mbarrier at `bar_cluster_addr`, a shared::cluster address that may belong to the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int c0, int c1, uint32_t bar_cluster_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void *dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar_cluster_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4,
                                                 uint32_t bar_cluster_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar_cluster_addr)
        : "memory");
}
// L2 eviction policies for the fp32 SwiGLU staging rows: they are read back exactly once, about one tile after they were
// written, while the operands of 74 other tiles stream through L2 in between.  Stored with evict_last and read back with
// evict_first, more of them are still in L2 when they are needed (less DRAM traffic; the time gained is within 1 %).
__device__ __forceinline__ uint64_t policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t policy_evict_last()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void st_global_v4_hint(float *a, const float4 v, uint64_t pol)
{
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "l"(pol) : "memory");
}
__device__ __forceinline__ float4 ld_global_cg_v4_hint(const float4 *a, uint64_t pol)
{
    float4 v;
    asm volatile("ld.global.cg.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(a), "l"(pol) : "memory");
    return v;
}
// shared::cluster address of `p` (a location in this CTA's shared memory) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void *p, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void prefetch_map(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols)
{
    if (CTAS == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {  // issued by the same warp of both CTAs of the pair, with the same shared-memory offset
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    if (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
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
// Pair forms.  The MMA reads A and its half of B from both CTAs' shared memory (same offsets) and writes each CTA's
// 128 accumulator rows to that CTA's TMEM.  The commit takes a shared::cluster address, so it can arrive on a
// barrier of either CTA; it is issued once per CTA of the pair.
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
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
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t layout_type = 2)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= layout_type << 61;  // 2 = 128-byte swizzle, 6 = 32-byte swizzle
    return d;
}

// Instruction descriptor for kind::i8: D = S32 (2 at bit 4), A = B = signed 8-bit (1 at bits 7 and 10),
// A K-major, B major per flag (bit 16), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(bool b_mn_major, int m)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------------------
// Tile schedule, rebuilt by every CTA from group_list (<= 1024 entries)
// ---------------------------------------------------------------------------------------------------------

// Row ranges follow GetSplitValueFromGroupList (gmm/grouped_matmul/op_kernel/grouped_matmul_utils.h:243-257):
// type 0 = running total, type 1 = count, values narrowed to int32; groups with no rows are skipped
// (grouped_matmul.h:263).  Ranges are clipped to [0, M] so a malformed list cannot address other memory.
__device__ void build_schedule(Shared *sh, const KParams &p, int tile_m)
{
    const int tid = threadIdx.x, L = p.gl_len;
    for (int g = tid; g < L; g += (int)blockDim.x) {
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
            if (p.part != 0) {
                // A 256-row tile on a trailing block of at most 128 rows would leave the second CTA of the pair idle:
                // the pair launch (part 1) stops short of such a block and a launch with 128-row tiles (part 2) takes it.
                const long long r = rows % (2 * BM);
                const bool small_tail = r > 0 && r <= BM;
                if (p.part == 1) { if (small_tail) rows -= r; }
                else if (small_tail) { start += rows - r; rows = r; }
                else rows = 0;
            }
            sh->row_start[g] = (int)start;
            sh->rows[g] = (int)rows;
            tsum += (int)((rows + tile_m - 1) / tile_m) * p.n_tiles;
        }
        int incl = tsum;
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        int run = incl - tsum;
        for (int g = lo; g < hi; ++g) {
            sh->tile_start[g] = run;
            run += ((sh->rows[g] + tile_m - 1) / tile_m) * p.n_tiles;
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

__device__ __forceinline__ Tile decode_tile(const Shared *sh, int t, int n_tiles, int L, int tile_m)
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
    tl.row0 = sh->row_start[lo] + mb * tile_m;
    tl.rows = min(tile_m, sh->rows[lo] - mb * tile_m);
    return tl;
}

// ---------------------------------------------------------------------------------------------------------
// Epilogue helpers
// ---------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float load_scale1(const void *p, int dtype, size_t i)
{
    if (dtype == kF32) return __ldg(reinterpret_cast<const float *>(p) + i);
    const uint16_t h = __ldg(reinterpret_cast<const uint16_t *>(p) + i);
    if (dtype == kBF16) return __uint_as_float((uint32_t)h << 16);
    return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // one cvt.rn.bf16x2.f32, round to nearest even
    return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi)
{
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// Four fp32 additions to 16 aligned bytes of global memory in one request, no value returned.
__device__ __forceinline__ void red_add_v4(float *p, const float4 v)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// q = int8(rint(half(S * (1 / (amax / 127)))))  -- CastFp32ToInt8Template,
// gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant_utils.h:308-316; NaN -> 0, saturating.
__device__ __forceinline__ uint32_t quant1(float s, float rcp)
{
    const __half h = __float2half_rn(__fmul_rn(s, rcp));
    const int q = max(-128, min(127, __half2int_rn(h)));
    return (uint32_t)q & 0xffu;
}
__device__ __forceinline__ uint32_t quant4(float4 v, float rcp)
{
    return quant1(v.x, rcp) | (quant1(v.y, rcp) << 8) | (quant1(v.z, rcp) << 16) | (quant1(v.w, rcp) << 24);
}

// Second half of grouped_matmul_swiglu_quant for rows [r_begin, r_end) of a finished row block (all of its N tiles
// have stored S and the row maxima): per row  qs = amax / 127, r = 1 / qs, q = int8(half(S * r))
// (gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant.h:496-503).  S and amax were written by
// other SMs, so they are read through L2 (ld.global.cg).  One warp per row.  Consecutive lanes read consecutive 16-byte
// pieces (a load instruction covers 512 contiguous bytes, a store 128): the tensor cores read their operands through the
// same shared-memory / L1 data path, so every extra line these accesses touch is taken from the MMAs.  Sixteen loads
// per lane are in flight at a time, because they wait for L2 under the full load of the GEMM.
__device__ void requant_rows(const KParams &p, int r_begin, int r_end, int warp_r, int lane)
{
    const int H = p.half_n;
    const int nf = H >> 2;  // 16-byte pieces per row
    const float *stage = reinterpret_cast<const float *>(p.out);
    for (int grow = r_begin + warp_r; grow < r_end; grow += EPI_WARPS) {
        const float amax = __uint_as_float(__ldcg(p.amax_bits + grow));
        const float4 *src = reinterpret_cast<const float4 *>(stage + (size_t)grow * H);
        uint32_t *dst = reinterpret_cast<uint32_t *>(p.q_out + (size_t)grow * H);
        float4 v[16];
        int f = lane;
        const uint64_t pol_first = policy_evict_first();
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = f + 32 * u < nf ? ld_global_cg_v4_hint(src + f + 32 * u, pol_first) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float qs = __fdiv_rn(amax, 127.0f);
        const float rcp = __fdiv_rn(1.0f, qs);
        if (lane == 0) p.q_scale_out[grow] = qs;
        while (true) {
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (f + 32 * u < nf) dst[f + 32 * u] = quant4(v[u], rcp);
            f += 512;
            if (f - lane >= nf) break;
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = f + 32 * u < nf ? ld_global_cg_v4_hint(src + f + 32 * u, pol_first) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
}

// Who requantises a finished row block, without any CTA ever waiting for another one (so the kernel does not depend on
// all CTAs being resident at the same time, nor on how many there are).
//
// Per row block two words in the workspace: state = arrivals (low 16 bits) + handed-over shares (high 16 bits), and a
// claim counter.  A block has `shares` contributors (N tiles x CTAs per tile) and is requantised in `shares` row slices.
//   * A CTA that has stored its part of the block "arrives" (atomic add of 1 after a fence).  The arrival that completes
//     the block takes one slice for itself plus one for every share handed over so far.
//   * Every other contributor keeps the block on a short pending list and looks at the state again after each of its
//     later tiles; once the block is complete it takes one slice.
//   * A contributor that cannot come back (its last tile is done, or its list is full) hands its share over with an
//     atomic add of 1 << 16.  If that add finds the block already complete it takes its slice itself; otherwise the
//     completing arrival, which comes later, sees the hand-over in the value its own add returns.
// Slices are claimed from the claim counter, so every slice is taken exactly once.
__device__ __forceinline__ void add_work(Shared *sh, int ws, int row0, int rows, int first, int count, int shares)
{
    const int k = sh->n_work[ws]++;
    sh->work_begin[ws][k] = row0 + (int)((long long)rows * first / shares);
    sh->work_end[ws][k] = row0 + (int)((long long)rows * (first + count) / shares);
}

__device__ __forceinline__ int ld_relaxed_gpu(const int *p)
{
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Publishing lane, after the whole CTA has stored a tile: arrive at block `rb`, look at the pending blocks, fill work list
// `ws`.  The caller fences before (release of the CTA's stores) and after (acquire of the other CTAs' stores).
__device__ void publish_and_collect(const KParams &p, Shared *sh, int ws, int rb, int row0, int rows, int shares)
{
    sh->n_work[ws] = 0;
    int *state = p.rb_counter;
    // the looks at the older blocks and the arrival travel together (one round trip to L2)
    int seen[MAX_PENDING];
#pragma unroll
    for (int i = 0; i < MAX_PENDING; ++i) seen[i] = i < sh->pend_n ? ld_relaxed_gpu(state + 2 * sh->pend_rb[i]) : 0;
    const int old = atomicAdd(state + 2 * rb, 1);
    const bool completed = (old & 0xffff) + 1 == shares;
    // slice claims, again together
    int first[MAX_PENDING];
#pragma unroll
    for (int i = 0; i < MAX_PENDING; ++i)
        first[i] = (i < sh->pend_n && (seen[i] & 0xffff) == shares) ? atomicAdd(state + 2 * sh->pend_rb[i] + 1, 1) : -1;
    const int cnt = 1 + (old >> 16);
    const int mine = completed ? atomicAdd(state + 2 * rb + 1, cnt) : -1;
    int n = 0;
#pragma unroll
    for (int i = 0; i < MAX_PENDING; ++i) {
        if (i >= sh->pend_n) break;
        if (first[i] >= 0) {
            add_work(sh, ws, sh->pend_row0[i], sh->pend_rows[i], first[i], 1, shares);
        } else {
            sh->pend_rb[n] = sh->pend_rb[i]; sh->pend_row0[n] = sh->pend_row0[i]; sh->pend_rows[n] = sh->pend_rows[i];
            ++n;
        }
    }
    sh->pend_n = n;
    if (completed) {
        add_work(sh, ws, row0, rows, mine, cnt, shares);
        return;
    }
    if (sh->pend_n == MAX_PENDING) {  // hand the oldest block's share over (or take it, if the block completed meanwhile)
        const int o = atomicAdd(state + 2 * sh->pend_rb[0], 1 << 16);
        if ((o & 0xffff) == shares)
            add_work(sh, ws, sh->pend_row0[0], sh->pend_rows[0], atomicAdd(state + 2 * sh->pend_rb[0] + 1, 1), 1, shares);
        for (int i = 1; i < MAX_PENDING; ++i) {
            sh->pend_rb[i - 1] = sh->pend_rb[i]; sh->pend_row0[i - 1] = sh->pend_row0[i]; sh->pend_rows[i - 1] = sh->pend_rows[i];
        }
        --sh->pend_n;
    }
    const int k = sh->pend_n++;
    sh->pend_rb[k] = rb; sh->pend_row0[k] = row0; sh->pend_rows[k] = rows;
}

// Publishing lane, after the CTA's last tile: every block still pending is taken once it is complete.  The other units
// are finishing at the same time, so the lane first looks on for up to `patience` cycles (nothing else is left to do;
// handing the share over at once would leave the last arrival of every block of the final wave with all of its slices,
// a serial tail of tens of microseconds); what is still incomplete after that is handed over, so the kernel never
// depends on the other CTAs being resident.
__device__ void release_pending(const KParams &p, Shared *sh, int ws, int shares, long long patience)
{
    sh->n_work[ws] = 0;
    int *state = p.rb_counter;
    const long long t0 = clock64();
    while (sh->pend_n > 0) {
        int n = 0;
        for (int i = 0; i < sh->pend_n; ++i) {
            if ((ld_relaxed_gpu(state + 2 * sh->pend_rb[i]) & 0xffff) == shares) {
                add_work(sh, ws, sh->pend_row0[i], sh->pend_rows[i], atomicAdd(state + 2 * sh->pend_rb[i] + 1, 1), 1, shares);
            } else {
                sh->pend_rb[n] = sh->pend_rb[i]; sh->pend_row0[n] = sh->pend_row0[i]; sh->pend_rows[n] = sh->pend_rows[i];
                ++n;
            }
        }
        sh->pend_n = n;
        if (n == 0 || clock64() - t0 > patience) break;
        __nanosleep(500);
    }
    for (int i = 0; i < sh->pend_n; ++i) {
        const int o = atomicAdd(state + 2 * sh->pend_rb[i], 1 << 16);
        if ((o & 0xffff) == shares)
            add_work(sh, ws, sh->pend_row0[i], sh->pend_rows[i], atomicAdd(state + 2 * sh->pend_rb[i] + 1, 1), 1, shares);
    }
    sh->pend_n = 0;
}

// Epilogue warp: requantise the row ranges of the next work list(s).  Every warp consumes every list, in order, and takes
// the rows warp, warp + EPI_WARPS, ... of each range.  With `blocking` unset only lists that are already written are
// taken; otherwise the call waits (bounded) for the next one.  Returns false when a wait gave up.
__device__ __forceinline__ bool consume_work(const KParams &p, Shared *sh, int &lists_done, int warp_e, int lane, bool blocking)
{
    while (true) {
        const int ws = lists_done % WK_DEPTH;
        const uint32_t parity = ((uint32_t)(lists_done / WK_DEPTH)) & 1u;
        int ready = 0;
        if (lane == 0) {
            ready = mbar_try_wait(smem_u32(&sh->wk_full[ws]), parity) ? 1 : 0;
            if (!ready && blocking) ready = mbar_wait(&sh->wk_full[ws], parity, sh, p.status, 650 + ws) ? 1 : -1;
        }
        ready = __shfl_sync(0xffffffffu, ready, 0);
        if (ready <= 0) return ready == 0;
        const int n = sh->n_work[ws];
        for (int k = 0; k < n; ++k) requant_rows(p, sh->work_begin[ws][k], sh->work_end[ws][k], warp_e, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->wk_empty[ws]);
        ++lists_done;
        if (blocking) return true;
    }
}

// ---------------------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------------------

// EPI selects the epilogue variant: kEpiPlain = no bias, no activation, per-token scale present, rows stored in place
// (the common case, compiled without per-element tests for the options); kEpiScatter = the same arithmetic with the
// result rows scattered through out_row_index, optionally into other GPUs' memory; kEpiGeneric = every option
// tested at run time.  CTAS: 1 = one CTA per tile, 2 = a cluster of two CTAs per 256-row tile.
template <int MODE, int BL, int EPI, int CTAS>
__global__ void __launch_bounds__(num_threads(MODE), 1)
gmm_w8a8_sm100_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const KParams p)
{
    constexpr bool B_MN_MAJOR = BL != kBTransposed;  // [E,K,N] and the fractal layout are N-contiguous
    constexpr bool PLAIN = EPI != kEpiGeneric;   // lean arithmetic
    constexpr bool SCATTER = EPI != kEpiPlain;  // rows go where out_row_index says
    constexpr bool COMBINE = EPI == kEpiCombine;  // fp32 rows combined into row_index[r] of a [out_rows, N] result
    using C = Cfg<CTAS>;
    constexpr int STAGES = C::kStages;
    constexpr int STAGE_BYTES = C::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    Shared *sh = reinterpret_cast<Shared *>(smem + PIPE_BYTES);
    // stage s: A at smem + s * STAGE_BYTES, weight box(es) right behind it

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = CTAS == 2 ? cluster_cta_rank() : 0u;  // position in the pair; rank 0 issues the MMAs
    const int unit = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;   // tile-processing unit (CTA or pair)
    const int n_units = CTAS == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sh->full[s], 1);   // pair: only rank 0's is used; its producer arrives, both CTAs' copies credit it
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh->acc_full[b], 1);
            mbar_init(&sh->acc_empty[b], EPI_WARPS * CTAS);  // one arrival per epilogue warp of every CTA of the unit
        }
        for (int b = 0; b < SCALE_BUFS; ++b) mbar_init(&sh->scale_ready[b], EPI_THREADS);
        for (int b = 0; b < WK_DEPTH; ++b) {
            mbar_init(&sh->wk_full[b], 1);
            mbar_init(&sh->wk_empty[b], EPI_WARPS);
        }
        sh->stored_count = 0;
        sh->abort_flag = 0;
        sh->total_tiles = 0;
        sh->wait_limit = p.wait_limit;
        sh->pend_n = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&map_x);
        prefetch_map(&map_w);
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(&sh->tmem_base, TMEM_COLS);
        tc_fence_before();
    }
    build_schedule(sh, p, C::kTileM);  // ends with __syncthreads()
    if (CTAS == 2) cluster_sync_all();  // the partner's barriers exist before anything is sent to them
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
            // pair: rank 0's full barriers as shared::cluster addresses (barriers are 8 bytes apart)
            const uint32_t full_rank0 = CTAS == 2 ? map_to_cta(&sh->full[0], 0) : 0u;
            // Pacing: the units of a wave (one round of the static schedule) share their operands through L2 - the N tiles
            // of a row block read the same rows of x, the row blocks of an expert the same weight boxes - and one launch
            // streams many times the L2's capacity, so a unit that drifts a tile or two away from the others finds the
            // shared data evicted and fetches it from DRAM again.  Every unit therefore announces the wave it starts and
            // waits, for at most about one tile's duration, until all units have started the wave before.  It is a hint,
            // never needed for correctness: when the wait runs out (units not resident together) pacing is switched off.
            bool pace = p.wave_cnt != nullptr && rank == 0;
            int wave = 0;
            for (int t = unit; t < total_tiles && ok; t += n_units, ++wave) {
                const Tile tl = decode_tile(sh, t, p.n_tiles, L, C::kTileM);
                // A CTA none of whose 128 rows belong to the group (the second CTA of a pair on a trailing block of at most
                // 128 rows) loads from beyond the last row of x instead: TMA then fills the box with zeros without touching
                // memory, and the tensor core multiplies zeros instead of the next group's rows (less traffic, less power;
                // the results of those rows are discarded either way).
                const int my_row0 = tl.rows > (int)rank * BM ? tl.row0 + (int)rank * BM : p.M;
                if (pace) {
                    if (wave > 0) {
                        const int expected = min(n_units, total_tiles - (wave - 1) * n_units);
                        const long long t0 = clock64();
                        while (ld_relaxed_gpu(p.wave_cnt + wave - 1) < expected) {
                            if (clock64() - t0 > p.pace_cycles) { pace = false; break; }
                            __nanosleep(500);
                        }
                    }
                    asm volatile("red.relaxed.gpu.global.add.s32 [%0], 1;" ::"l"(p.wave_cnt + wave) : "memory");
                }
                int n0, n1;
                if (MODE == kModeSwigluQuant) { n0 = tl.n_idx * (BN / 2); n1 = p.half_n + n0; }
                else { n0 = tl.n_idx * BN; n1 = n0 + BN / 2; }
                const int nb = rank == 0 ? n0 : n1;  // pair: the weight box this CTA contributes
                // test hook: leaving K blocks out of the last tile makes the MMA issuer's wait run out (nothing else is touched)
                const int kb_end = p.num_k_blocks - (t + n_units >= total_tiles ? p.skip_k_blocks : 0);
                for (int kb = 0; kb < kb_end; ++kb) {
                    if (!mbar_wait(&sh->empty[stage], phase ^ 1u, sh, p.status, 100 + stage)) { ok = false; break; }
                    uint8_t *adst = smem + stage * STAGE_BYTES;
                    uint8_t *bdst = adst + A_STAGE;
                    if (CTAS == 1) {
                        mbar_arrive_expect_tx(&sh->full[stage], C::kTxBytes);
                        tma_load_2d(adst, &map_x, kb * BK, my_row0, &sh->full[stage]);
                        if (BL == kBFractalNz) {  // map dims {32 n, 16 k, K/16, N/32, E}: a box is 128 k x 128 n in 32-column slabs
                            tma_load_5d(bdst, &map_w, 0, 0, kb * (BK / 16), n0 >> 5, tl.g, &sh->full[stage]);
                            tma_load_5d(bdst + B_BOX, &map_w, 0, 0, kb * (BK / 16), n1 >> 5, tl.g, &sh->full[stage]);
                        } else if (B_MN_MAJOR) {  // weight [E, K, N]: map dims {N, K, E}
                            tma_load_3d(bdst, &map_w, n0, kb * BK, tl.g, &sh->full[stage]);
                            tma_load_3d(bdst + B_BOX, &map_w, n1, kb * BK, tl.g, &sh->full[stage]);
                        } else {           // weight [E, N, K]: map dims {K, N, E}
                            tma_load_3d(bdst, &map_w, kb * BK, n0, tl.g, &sh->full[stage]);
                            tma_load_3d(bdst + B_BOX, &map_w, kb * BK, n1, tl.g, &sh->full[stage]);
                        }
                    } else {
                        if (rank == 0) mbar_arrive_expect_tx(&sh->full[stage], C::kTxBytes);
                        tma_load_2d_pair(adst, &map_x, kb * BK, my_row0, full_rank0 + (uint32_t)stage * 8u);
                        if (BL == kBFractalNz) tma_load_5d_pair(bdst, &map_w, 0, 0, kb * (BK / 16), nb >> 5, tl.g, full_rank0 + (uint32_t)stage * 8u);
                        else if (B_MN_MAJOR) tma_load_3d_pair(bdst, &map_w, nb, kb * BK, tl.g, full_rank0 + (uint32_t)stage * 8u);
                        else tma_load_3d_pair(bdst, &map_w, kb * BK, nb, tl.g, full_rank0 + (uint32_t)stage * 8u);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if ((!ok || *(volatile int *)&sh->abort_flag) && rank == 0) {
                // Drain: give the copies already issued a bounded chance to land before the CTA leaves.
                const int n = (int)(issued < STAGES ? issued : STAGES);
                int s2 = stage;
                uint32_t ph = phase;
                for (int i = 0; i < n; ++i) {
                    if (--s2 < 0) { s2 = STAGES - 1; ph ^= 1u; }
                    const uint32_t a = smem_u32(&sh->full[s2]);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(a, ph) && clock64() - t0 < DRAIN_LIMIT_CYCLES) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (rank 0 of the unit) ------------------------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(B_MN_MAJOR, C::kTileM);
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const uint32_t empty_peer = CTAS == 2 ? map_to_cta(&sh->empty[0], 1) : 0u;       // the partner's barriers
            const uint32_t acc_full_peer = CTAS == 2 ? map_to_cta(&sh->acc_full[0], 1) : 0u;
            int ti = 0;
            TRACE_GT(0, 0, 0);
            for (int t = unit; t < total_tiles && ok; t += n_units, ++ti) {
                TRACE(1, ti, 0);
                if (!mbar_wait(&sh->acc_empty[buf], acc_phase ^ 1u, sh, p.status, 200 + buf)) { ok = false; break; }
                TRACE(1, ti, 1);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    if (!mbar_wait(&sh->full[stage], phase, sh, p.status, 300 + stage)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_STAGE;
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        const uint64_t a_desc = make_smem_desc(a_addr + j * UMMA_K, 16, 1024);
                        // [E,K,N]: 128-byte runs along N, 8 K-rows = 1024 B, next 128 columns one box on.
                        // fractal: 32-byte runs along N, 8 K-rows = 256 B, next 32 columns 128 K-rows (4096 B) on.
                        const uint64_t b_desc = BL == kBFractalNz ? make_smem_desc(b_addr + j * UMMA_K * 32, 4096, 256, 6)
                                                : B_MN_MAJOR      ? make_smem_desc(b_addr + j * UMMA_K * 128, B_BOX, 1024)
                                                                  : make_smem_desc(b_addr + j * UMMA_K, 16, 1024);
                        if (CTAS == 1) umma_i8(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
                        else umma_i8_pair(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    if (CTAS == 1) {
                        umma_commit(&sh->empty[stage]);
                    } else {  // the stage is free in both CTAs once these MMAs have read it
                        umma_commit_pair(smem_u32(&sh->empty[stage]));
                        umma_commit_pair(empty_peer + (uint32_t)stage * 8u);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                TRACE(1, ti, 2);
                TRACE_GT(0, 0, 1);
                if (CTAS == 1) {
                    umma_commit(&sh->acc_full[buf]);
                } else {
                    umma_commit_pair(smem_u32(&sh->acc_full[buf]));
                    umma_commit_pair(acc_full_peer + (uint32_t)buf * 8u);
                }
                buf ^= 1;
                if (buf == 0) acc_phase ^= 1u;
            }
        }
    } else if (warp < 2 + EPI_WARPS) {
        // ------------------------------ epilogue: warp -> (TMEM lane quarter, column half) ------------------------------
        const int quarter = warp & 3;
        const int chalf = (warp - 2) >> 2;
        const int te = (int)threadIdx.x - 64;  // 0 .. EPI_THREADS-1
        const int r = quarter * 32 + lane;     // row inside the tile == TMEM lane
        uint8_t *my_stage = sh->out_stage[warp - 2];
        int buf = 0, it = 0;
        uint32_t acc_phase = 0;
        int lists_done = 0, lists_total = 0;
        const uint64_t pol_last = policy_evict_last();
        const uint32_t acc_empty_rank0 = CTAS == 2 ? map_to_cta(&sh->acc_empty[0], 0) : 0u;
        for (int t = unit; t < total_tiles; t += n_units, ++it) {
            const Tile tl = decode_tile(sh, t, p.n_tiles, L, C::kTileM);
            const int my_row0 = tl.row0 + (int)rank * BM;                 // this CTA's 128 rows of the tile
            const int my_rows = max(0, min(BM, tl.rows - (int)rank * BM));
            const bool valid = r < my_rows;
            const bool warp_has_rows = quarter * 32 < my_rows;
            const int grow = my_row0 + r;
            const size_t sbase = (size_t)tl.g * p.N;
            const int n0 = MODE == kModeSwigluQuant ? tl.n_idx * (BN / 2) : tl.n_idx * BN;

            // Stage this tile's per-column scales in shared memory; the loads overlap the wait for the MMAs.
            const int sb = it % SCALE_BUFS;
            if (MODE != kModeInt32) {
                int col;
                bool in_range;
                if (MODE == kModeSwigluQuant) {
                    const int j = te < BN / 2 ? te : te - BN / 2;
                    in_range = n0 + j < p.half_n;
                    col = (te < BN / 2 ? 0 : p.half_n) + n0 + j;
                } else {
                    col = n0 + te;
                    in_range = col < p.N;
                }
                sh->scales[sb][te] = in_range ? load_scale1(p.w_scale, p.w_scale_dtype, sbase + col) : 0.0f;
                mbar_arrive(&sh->scale_ready[sb]);
            }
            const float xs = (valid && p.x_scale) ? __ldg(p.x_scale + grow) : 1.0f;
            long long out_row = grow;
            float lg = 1.0f;
            if (COMBINE) {
                out_row = -1;
                if (valid) {
                    out_row = p.row_index_i32 ? (long long)__ldg(reinterpret_cast<const int *>(p.row_index) + grow)
                                              : __ldg(reinterpret_cast<const long long *>(p.row_index) + grow);
                    if (p.logit) lg = __ldg(p.logit + grow);
                }
            } else if (MODE != kModeSwigluQuant && SCATTER && p.out_row_index && valid) out_row = __ldg(p.out_row_index + grow);
            if (te == 0) TRACE(2, it, 0);
            if (MODE != kModeInt32 && !mbar_wait(&sh->scale_ready[sb], (uint32_t)(it / SCALE_BUFS) & 1u, sh, p.status, 500 + sb)) break;
            if (!mbar_wait(&sh->acc_full[buf], acc_phase, sh, p.status, 400 + buf)) break;
            if (te == 0) TRACE(2, it, 1);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * BN;
            const float *tsc = sh->scales[sb];

            if (warp_has_rows) {
                if (MODE == kModeSwigluQuant) {
                    float amax = 0.0f;
                    float *sout = reinterpret_cast<float *>(p.out);
#pragma unroll 1
                    for (int c = chalf * 2; c < chalf * 2 + 2; ++c) {
                        if (n0 + c * 32 >= p.half_n) break;
                        uint32_t va[32], vb[32];
                        tmem_ld32(taddr + c * 32, va);
                        tmem_ld32(taddr + BN / 2 + c * 32, vb);
                        tmem_ld_wait();
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 sa = *reinterpret_cast<const float4 *>(tsc + c * 32 + j4 * 4);
                            const float4 sg = *reinterpret_cast<const float4 *>(tsc + BN / 2 + c * 32 + j4 * 4);
                            const float sav[4] = {sa.x, sa.y, sa.z, sa.w}, sgv[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                // (acc * x_scale) * w_scale, then S = gate * (act / (1 + exp(-act)))
                                const float a = __fmul_rn(__fmul_rn(__int2float_rn((int)va[j4 * 4 + j]), xs), sav[j]);
                                const float b = __fmul_rn(__fmul_rn(__int2float_rn((int)vb[j4 * 4 + j]), xs), sgv[j]);
                                const float den = __fadd_rn(1.0f, expf(-a));
                                const float sw = __fdiv_rn(a, den);
                                const float sv = __fmul_rn(b, sw);
                                va[j4 * 4 + j] = __float_as_uint(sv);
                                if (n0 + c * 32 + j4 * 4 + j < p.half_n) amax = fmaxf(amax, fabsf(sv));
                            }
                        }
                        // Transpose through shared memory, 16 rows per round, so that eight lanes store 128 contiguous bytes
                        // of one row of S: a store instruction then touches 4 lines instead of 32 (the shared-memory / L1
                        // data path is the one the tensor cores read their operands through).
                        const int pc = lane & 7;
                        const int col = n0 + c * 32 + pc * 4;
#pragma unroll
                        for (int round = 0; round < 2; ++round) {
                            if ((lane >> 4) == round) {
#pragma unroll
                                for (int q8 = 0; q8 < 8; ++q8)
                                    *reinterpret_cast<uint4 *>(my_stage + (lane & 15) * 128 + (((q8 ^ lane) & 7) << 4)) =
                                        make_uint4(va[q8 * 4], va[q8 * 4 + 1], va[q8 * 4 + 2], va[q8 * 4 + 3]);
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int r16 = i * 4 + (lane >> 3);
                                const int rr = quarter * 32 + round * 16 + r16;
                                const float4 val = *reinterpret_cast<const float4 *>(my_stage + r16 * 128 + (((pc ^ r16) & 7) << 4));
                                if (rr < my_rows && col < p.half_n)
                                    st_global_v4_hint(sout + (size_t)(my_row0 + rr) * p.half_n + col, val, pol_last);
                            }
                            __syncwarp();
                        }
                    }
                    if (valid) atomicMax(p.amax_bits + grow, __float_as_uint(amax));
                } else if (MODE == kModeInt32) {
#pragma unroll 1
                    for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
                        if (n0 + c * 32 >= p.N) break;
                        uint32_t v[32];
                        tmem_ld32(taddr + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const int col = n0 + c * 32 + j4 * 4;
                            if (col < p.N && valid && (!SCATTER || (out_row >= 0 && (p.out_rows <= 0 || out_row < p.out_rows)))) {
                                int acc[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    acc[j] = (int)v[j4 * 4 + j];
                                    if (!PLAIN && p.bias_dtype == kI32) acc[j] += __ldg(reinterpret_cast<const int *>(p.bias) + sbase + col + j);
                                }
                                *reinterpret_cast<int4 *>(reinterpret_cast<int *>(p.out) + (size_t)out_row * p.N + col) =
                                    make_int4(acc[0], acc[1], acc[2], acc[3]);
                            }
                        }
                    }
                } else if (COMBINE) {
                    // grouped_matmul_finalize_routing: t = float(acc) * scale[n]; t *= (per_token[m] * logit[m]);
                    // t += logit[m] * float(bias[n]); y[row_index[m], n] += t  (ComputeDequantAndActivate,
                    // DataCopyPerTokenScaleAndBrcb, VectorAtomicProcess of
                    // gmm/grouped_matmul_finalize_routing/op_kernel/grouped_matmul_finalize_routing.h:418-448, 497-545, 343-366).
                    float *out = reinterpret_cast<float *>(p.out);
                    const float rs = p.logit ? (p.x_scale ? __fmul_rn(xs, lg) : lg) : xs;
                    // One 32-column chunk at a time: 32 fp32 = 128 bytes per row and pass.
#pragma unroll 1
                    for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
                        if (n0 + c * 32 >= p.N) break;
                        uint32_t v[32], pk[32];
                        tmem_ld32(taddr + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 s4 = *reinterpret_cast<const float4 *>(tsc + c * 32 + j4 * 4);
                            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int cc = c * 32 + j4 * 4 + j;
                                float tv = __fmul_rn(__fmul_rn(__int2float_rn((int)v[j4 * 4 + j]), sv[j]), rs);
                                if (p.bias_dtype == kBF16 && n0 + cc < p.N) {
                                    const float b = __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t *>(p.bias) + sbase + n0 + cc) << 16);
                                    tv = __fadd_rn(tv, __fmul_rn(lg, b));
                                }
                                pk[j4 * 4 + j] = __float_as_uint(tv);
                            }
                        }
                        // Same transposition as the bf16 path: eight lanes then hold 128 contiguous bytes of one row, so a
                        // vector reduction covers whole 32-byte sectors of the fp32 result.
                        const int pc = lane & 7;
                        const int col = n0 + c * 32 + pc * 4;
#pragma unroll
                        for (int round = 0; round < 2; ++round) {
                            if ((lane >> 4) == round) {
#pragma unroll
                                for (int q8 = 0; q8 < 8; ++q8)
                                    *reinterpret_cast<uint4 *>(my_stage + (lane & 15) * 128 + (((q8 ^ lane) & 7) << 4)) =
                                        make_uint4(pk[q8 * 4], pk[q8 * 4 + 1], pk[q8 * 4 + 2], pk[q8 * 4 + 3]);
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int r16 = i * 4 + (lane >> 3);
                                const int rr = round * 16 + r16;
                                const float4 val = *reinterpret_cast<const float4 *>(my_stage + r16 * 128 + (((pc ^ r16) & 7) << 4));
                                const long long orow = __shfl_sync(0xffffffffu, out_row, rr);
                                if (quarter * 32 + rr < my_rows && col < p.N && orow >= 0 && orow < p.out_rows) {
                                    float *dst = out + (size_t)orow * p.N + col;
                                    if (p.scatter_add) red_add_v4(dst, val);
                                    else *reinterpret_cast<float4 *>(dst) = val;
                                }
                            }
                            __syncwarp();
                        }
                    }
                } else {
                    uint16_t *out = reinterpret_cast<uint16_t *>(p.out);
                    // Two 32-column chunks at a time: 64 bf16 = 128 bytes per row and pass.
#pragma unroll 1
                    for (int c = chalf * 4; c < chalf * 4 + 4; c += 2) {
                        if (n0 + c * 32 >= p.N) break;
                        uint32_t pk[32];
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            uint32_t v[32];
                            tmem_ld32(taddr + (c + half) * 32, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int j4 = 0; j4 < 8; ++j4) {
                                const float4 s4 = *reinterpret_cast<const float4 *>(tsc + (c + half) * 32 + j4 * 4);
                                const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
                                float o[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    // (acc * w_scale) * x_scale, optional bf16 bias, optional relu, then bf16 RNE
                                    const int cc = (c + half) * 32 + j4 * 4 + j;
                                    int acc = (int)v[j4 * 4 + j];
                                    if (PLAIN) {
                                        o[j] = __fmul_rn(__fmul_rn(__int2float_rn(acc), sv[j]), xs);
                                    } else {
                                        const bool in_n = n0 + cc < p.N;
                                        if (p.bias_dtype == kI32 && in_n) acc += __ldg(reinterpret_cast<const int *>(p.bias) + sbase + n0 + cc);
                                        float tv = __fmul_rn(__int2float_rn(acc), sv[j]);
                                        if (p.x_scale) tv = __fmul_rn(tv, xs);
                                        if (p.bias_dtype == kBF16 && in_n)
                                            tv = __fadd_rn(tv, __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t *>(p.bias) + sbase + n0 + cc) << 16));
                                        tv = apply_activation(p.act_type, tv);
                                        o[j] = tv;
                                    }
                                }
                                if (!PLAIN && p.out_f16) {
                                    pk[half * 16 + j4 * 2] = pack_f16x2(o[0], o[1]);
                                    pk[half * 16 + j4 * 2 + 1] = pack_f16x2(o[2], o[3]);
                                } else {
                                    pk[half * 16 + j4 * 2] = pack_bf16x2(o[0], o[1]);
                                    pk[half * 16 + j4 * 2 + 1] = pack_bf16x2(o[2], o[3]);
                                }
                            }
                        }
                        // Transpose through shared memory, 16 rows per round, so that eight lanes write 128 contiguous
                        // bytes of one row (a full line for local memory, a full-size packet for a peer GPU).
                        const int pc = lane & 7;
                        const int col = n0 + c * 32 + pc * 8;
#pragma unroll
                        for (int round = 0; round < 2; ++round) {
                            if ((lane >> 4) == round) {
#pragma unroll
                                for (int q8 = 0; q8 < 8; ++q8)
                                    *reinterpret_cast<uint4 *>(my_stage + (lane & 15) * 128 + (((q8 ^ lane) & 7) << 4)) =
                                        make_uint4(pk[q8 * 4], pk[q8 * 4 + 1], pk[q8 * 4 + 2], pk[q8 * 4 + 3]);
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int r16 = i * 4 + (lane >> 3);
                                const int rr = round * 16 + r16;
                                const uint4 val = *reinterpret_cast<const uint4 *>(my_stage + r16 * 128 + (((pc ^ r16) & 7) << 4));
                                long long orow = my_row0 + quarter * 32 + rr;
                                uint16_t *obase = out;
                                bool in_rows = quarter * 32 + rr < my_rows;
                                if (SCATTER) {
                                    orow = __shfl_sync(0xffffffffu, out_row, rr);
                                    long long gpu_field = 0;
                                    if (p.num_peers > 0) {  // high bits: which GPU's buffer, low 40 bits: row in it
                                        gpu_field = orow >> 40;
                                        orow &= (1ll << 40) - 1;
                                    }
                                    // an index that names no peer or no row of the result is skipped and reported, not stored
                                    if (in_rows && (orow < 0 || gpu_field >= (p.num_peers > 0 ? p.num_peers : 1) || (p.out_rows > 0 && orow >= p.out_rows))) {
                                        if (pc == 0 && c == chalf * 4 && atomicCAS(p.status, kStatusOk, kStatusBadIndex) == kStatusOk) {
                                            p.status[1] = (int)blockIdx.x;
                                            p.status[2] = 800;
                                            p.status[3] = my_row0 + quarter * 32 + rr;
                                        }
                                        in_rows = false;
                                    } else if (p.num_peers > 0) {
                                        obase = reinterpret_cast<uint16_t *>(p.out_peers[(int)gpu_field]);
                                    }
                                }
                                if (in_rows && col < p.N) *reinterpret_cast<uint4 *>(obase + (size_t)orow * p.N + col) = val;
                            }
                            __syncwarp();
                        }
                    }
                }
            }
            if (te == 0) TRACE(2, it, 2);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {  // the accumulator buffer may be overwritten once every epilogue warp of the unit has read it
                if (CTAS == 1) mbar_arrive(&sh->acc_empty[buf]);
                else mbar_arrive_cluster(acc_empty_rank0 + (uint32_t)buf * 8u);
            }
            buf ^= 1;
            if (buf == 0) acc_phase ^= 1u;

            if (MODE == kModeSwigluQuant) {
                // Tell the publishing lane that this thread's part of the tile is stored (the fence orders the stores and
                // the row maximum before the count), then take the work list it writes for this tile.  That list comes
                // within a few round trips to L2 (the lane waits for no other CTA) and names the row blocks that are
                // complete by now - normally the block of this unit's previous tile, whose rows are then read while
                // they are still in L2; one tile later they would have been evicted.
                __threadfence();
                if (te == 0) TRACE(2, it, 3);
                atomicAdd(&sh->stored_count, 1u);
                if (!consume_work(p, sh, lists_done, warp - 2, lane, true)) break;
                if (te == 0) { TRACE(2, it, 4); TRACE_ADD(2, it, 5, lists_done); }
            }
        }
        if (MODE == kModeSwigluQuant && !*(volatile int *)&sh->abort_flag) {
            // one list per tile of this unit plus the closing one: wait (bounded) for those not seen yet
            lists_total = it + 1;
            while (lists_done < lists_total)
                if (!consume_work(p, sh, lists_done, warp - 2, lane, true)) break;
        }
        if (SCATTER && p.num_peers > 0) __threadfence_system();  // rows stored into other GPUs' memory
    }

    else if (MODE == kModeSwigluQuant) {
        // ------------------------------ publishing lane (swiglu_quant) ------------------------------
        // Per tile of this unit, in the epilogue's order: wait until every epilogue thread has stored the tile, arrive at its
        // row block, collect the row slices that fall to this CTA now (publish_and_collect) into the next work list.  After
        // the last tile one more list takes or hands over what is still pending.  Nothing here waits for another CTA; the
        // only back-pressure is the ring of work lists, which the epilogue warps empty after every tile.
        if (lane == 0) {
            const int shares = p.n_tiles * CTAS;
            int it = 0;
            bool ok = true;
            for (int t = unit; t < total_tiles && ok; t += n_units, ++it) {
                const int ws = it % WK_DEPTH;
                const unsigned need = (unsigned)(it + 1) * EPI_THREADS;
                if (*(volatile unsigned *)&sh->stored_count < need) {
                    const long long t0 = clock64();
                    while (*(volatile unsigned *)&sh->stored_count < need) {
                        __nanosleep(200);
                        if (*(volatile int *)&sh->abort_flag) { ok = false; break; }
                        if (clock64() - t0 > sh->wait_limit) {
                            *(volatile int *)&sh->abort_flag = 1;
                            if (atomicCAS(p.status, kStatusOk, kStatusWaitTimeout) == kStatusOk) {
                                p.status[1] = (int)blockIdx.x;
                                p.status[2] = 620;
                                p.status[3] = it;
                            }
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                }
                TRACE(3, it, 0);
                if (!mbar_wait(&sh->wk_empty[ws], (((uint32_t)(it / WK_DEPTH)) & 1u) ^ 1u, sh, p.status, 630 + ws)) { ok = false; break; }
                const Tile tl = decode_tile(sh, t, p.n_tiles, L, C::kTileM);
                TRACE(3, it, 1);
                __threadfence();
                publish_and_collect(p, sh, ws, p.rb_base + t / p.n_tiles, tl.row0, tl.rows, shares);
                __threadfence();
                TRACE(3, it, 2);
                TRACE_ADD(3, it, 3, sh->n_work[ws]);
                mbar_arrive(&sh->wk_full[ws]);
            }
            if (ok && !*(volatile int *)&sh->abort_flag) {
                const int ws = it % WK_DEPTH;
                if (mbar_wait(&sh->wk_empty[ws], (((uint32_t)(it / WK_DEPTH)) & 1u) ^ 1u, sh, p.status, 640 + ws)) {
                    release_pending(p, sh, ws, shares, 2ll * p.pace_cycles);
                    __threadfence();
                    mbar_arrive(&sh->wk_full[ws]);
                }
            }
        }
    }

    __syncthreads();
    if (CTAS == 2) cluster_sync_all();  // neither CTA leaves, or frees TMEM, while the other can still reach into it
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, TMEM_COLS);
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

template <int MODE, int BL, int EPI, int CTAS>
cudaError_t launch_variant(const Plan &plan, const KParams &kp, cudaStream_t stream)
{
    auto kern = gmm_w8a8_sm100_kernel<MODE, BL, EPI, CTAS>;
    // Once per device and instantiation; the attribute is idempotent, so a race only repeats the call.
    static unsigned long long done_mask = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!((done_mask >> (dev & 63)) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return e;
        done_mask |= 1ull << (dev & 63);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(CTAS == 2 ? (plan.num_sms & ~1) : plan.num_sms), 1, 1);
    cfg.blockDim = dim3(num_threads(MODE), 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = CTAS == 2 ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, plan.map_x, plan.map_w, kp);
}

template <int MODE, int BL, int EPI>
cudaError_t launch_ctas(const Plan &plan, const KParams &kp, cudaStream_t stream)
{
    return plan.ctas == 2 ? launch_variant<MODE, BL, EPI, 2>(plan, kp, stream) : launch_variant<MODE, BL, EPI, 1>(plan, kp, stream);
}

template <int MODE, int BL>
cudaError_t launch_epi(int epi, const Plan &plan, const KParams &kp, cudaStream_t stream)
{
    if (MODE == kModeSwigluQuant || epi == kEpiPlain) return launch_ctas<MODE, BL, kEpiPlain>(plan, kp, stream);
    if (epi == kEpiScatter) return launch_ctas<MODE, BL, kEpiScatter>(plan, kp, stream);
    if (MODE == kModeDequantBf16 && epi == kEpiCombine) return launch_ctas<MODE, BL, MODE == kModeDequantBf16 ? kEpiCombine : kEpiPlain>(plan, kp, stream);
    return launch_ctas<MODE, BL, kEpiGeneric>(plan, kp, stream);
}

template <int MODE>
cudaError_t launch_layout(int layout, int epi, const Plan &plan, const KParams &kp, cudaStream_t stream)
{
    if (layout == kBTransposed) return launch_epi<MODE, kBTransposed>(epi, plan, kp, stream);
    if (layout == kBFractalNz) return launch_epi<MODE, kBFractalNz>(epi, plan, kp, stream);
    return launch_epi<MODE, kBRowMajor>(epi, plan, kp, stream);
}

}  // namespace

// The tcgen05 path needs 16-byte aligned row pitches for TMA (K for x; N or K for the weight), 16-byte
// aligned base pointers and, for SwiGLU, a half width that keeps the second box aligned.
bool sm100_shape_ok(const Problem &p)
{
    if (p.K % 16 != 0 || p.N % 16 != 0) return false;
    if (p.mode == kModeSwigluQuant && p.N % 32 != 0) return false;
    if (p.w_layout == kBFractalNz && (p.N % 32 != 0 || (p.mode == kModeSwigluQuant && p.N % 64 != 0))) return false;
    if (p.gl_len > MAX_GROUPS || p.gl_len <= 0) return false;
    if (p.M <= 0 || p.M > 0x7fffffffll / 2 || p.K > 0x7fffffffll || p.N > 0x7fffffffll) return false;
    if ((reinterpret_cast<uintptr_t>(p.x) & 15) || (reinterpret_cast<uintptr_t>(p.w) & 15)) return false;
    if (reinterpret_cast<uintptr_t>(p.out0) & 15) return false;
    if (reinterpret_cast<uintptr_t>(p.w_scale) & 3) return false;
    if (p.bias && (reinterpret_cast<uintptr_t>(p.bias) & 3)) return false;
    if (p.mode == kModeSwigluQuant && (!p.out1 || (reinterpret_cast<uintptr_t>(p.out1) & 3))) return false;
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
    if (p.w_layout == kBFractalNz) {
        // FRACTAL_NZ [E, N/32, K/16, 16, 32]: element (k, n) at ((n/32 * K/16 + k/16) * 16 + k%16) * 32 + n%32
        cuuint64_t dims[5] = {32, 16, (cuuint64_t)(p.K / 16), (cuuint64_t)(p.N / 32), (cuuint64_t)p.E};
        cuuint64_t strides[4] = {32, 512, (cuuint64_t)p.K * 32, (cuuint64_t)p.K * (cuuint64_t)p.N};
        cuuint32_t box[5] = {32, 16, BK / 16, 4, 1};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUresult r = enc(&plan.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<int8_t *>(p.w), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    } else {
        const bool tr = p.w_layout == kBTransposed;
        const cuuint64_t inner = tr ? p.K : p.N, mid = tr ? p.N : p.K;
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
    plan.num_sms = device_sm_count();
    if (plan.num_sms <= 0) return cudaErrorNoDevice;
    if (p.opt.max_ctas > 0 && p.opt.max_ctas < plan.num_sms) plan.num_sms = p.opt.max_ctas;
    if (plan.num_sms < 2) {  // a CTA pair needs two CTAs
        plan.ctas = 1;
        plan.hybrid = false;
    }
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    KParams kp;
    kp.group_list = p.group_list;
    kp.gl_len = p.gl_len;
    kp.gl_type = p.gl_type;
    kp.M = (int)p.M;
    kp.K = (int)p.K;
    kp.N = (int)p.N;
    kp.half_n = (int)(p.N / 2);
    if (plan.ctas != 2) plan.ctas = 1;
    kp.n_tiles = p.mode == kModeSwigluQuant ? (int)((p.N / 2 + BN / 2 - 1) / (BN / 2)) : (int)((p.N + BN - 1) / BN);
    kp.num_k_blocks = (int)((p.K + BK - 1) / BK);
    kp.w_scale = p.w_scale;
    kp.w_scale_dtype = p.w_scale_dtype;
    kp.x_scale = p.x_scale;
    kp.bias = p.bias;
    kp.bias_dtype = p.bias ? p.bias_dtype : kNone;
    kp.act_type = p.act_type;
    kp.out_f16 = p.out_f16;
    kp.status = reinterpret_cast<int *>(ws + plan.off_status);
    kp.amax_bits = reinterpret_cast<unsigned *>(ws + plan.off_amax);
    kp.rb_counter = reinterpret_cast<int *>(ws + plan.off_done);
    kp.out_row_index = reinterpret_cast<const long long *>(p.out_row_index);
    kp.q_out = reinterpret_cast<int8_t *>(p.out0);
    kp.q_scale_out = reinterpret_cast<float *>(p.out1);
    kp.out = p.mode == kModeSwigluQuant ? static_cast<void *>(ws + plan.off_stage) : p.out0;

    cudaError_t e;
    const bool lean = !p.bias && p.act_type == 0 && !p.out_f16 && (p.mode != kModeDequantBf16 || p.x_scale);
    const int epi = p.combine ? kEpiCombine : !lean ? kEpiGeneric : (p.out_row_index ? kEpiScatter : kEpiPlain);
    kp.logit = p.logit;
    kp.row_index = p.row_index;
    kp.row_index_i32 = p.row_index_i32;
    kp.scatter_add = p.scatter_add;
    kp.out_rows = p.out_rows;
    if (p.combine && (p.mode != kModeDequantBf16 || !p.row_index)) return cudaErrorInvalidValue;
    kp.num_peers = p.mode == kModeDequantBf16 ? p.num_peers : 0;
    for (int i = 0; i < 8; ++i) kp.out_peers[i] = i < kp.num_peers ? p.out_peers[i] : nullptr;
    if (kp.num_peers > 0 && epi != kEpiScatter) return cudaErrorInvalidValue;
    // Pacing (see the producer): needs one zeroed word per wave; the plan reserves them only where it pays.
    kp.wave_cnt = plan.off_wave ? reinterpret_cast<int *>(ws + plan.off_wave) : nullptr;
    kp.pace_cycles = kp.num_k_blocks * 1200 + 20000;   // about one tile's duration
#ifdef GMM_TRACE
    kp.trace = getenv("GMM_TRACE_PTR") ? reinterpret_cast<long long *>(strtoull(getenv("GMM_TRACE_PTR"), nullptr, 0)) : nullptr;
#endif
    if (const char *e = getenv("GMM_B200_PACE")) {
        if (e[0] == '0') kp.wave_cnt = nullptr;
        else if (atoi(e) > 1) kp.pace_cycles = atoi(e);
    }
    kp.wait_limit = p.opt.wait_limit_cycles > 0 ? p.opt.wait_limit_cycles : WAIT_LIMIT_CYCLES;
    kp.skip_k_blocks = p.opt.test_skip_k_blocks > 0 ? (p.opt.test_skip_k_blocks < kp.num_k_blocks ? p.opt.test_skip_k_blocks : kp.num_k_blocks) : 0;
    if (p.opt.ev_start) cudaEventRecord(p.opt.ev_start, stream);
    // Pair tiles for the bulk of every group, then (plan.hybrid) 128-row tiles for the trailing blocks a pair would half waste.
    const int launches = plan.ctas == 2 && plan.hybrid ? 2 : 1;
    Plan one = plan;
    for (int i = 0; i < launches; ++i) {
        kp.part = launches == 2 ? i + 1 : 0;
        kp.rb_base = i == 0 ? 0 : (int)((p.M + 2 * BM - 1) / (2 * BM)) + p.gl_len + 1;
        const Plan &pl = i == 0 ? plan : one;
        if (i == 1) {
            one.ctas = 1;
            kp.wave_cnt = nullptr;  // the pacing counters belong to the first launch
        }
        if (p.mode == kModeSwigluQuant) e = launch_layout<kModeSwigluQuant>(p.w_layout, epi, pl, kp, stream);
        else if (p.mode == kModeInt32) e = launch_layout<kModeInt32>(p.w_layout, epi, pl, kp, stream);
        else e = launch_layout<kModeDequantBf16>(p.w_layout, epi, pl, kp, stream);
        if (e != cudaSuccess) break;
    }
    if (p.opt.ev_stop) cudaEventRecord(p.opt.ev_stop, stream);
    return e;
}

}  // namespace gmm
