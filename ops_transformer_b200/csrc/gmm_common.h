// Internal interface between the aclnn-compatible host layer and the CUDA launchers.
// Nothing here is exported; the public C ABI lives in include/.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <vector>

namespace gmm {

// Data-type codes follow aclDataType (include/aclnn/aclnn_base.h).
enum : int { kF32 = 0, kF16 = 1, kI8 = 2, kI32 = 3, kI64 = 9, kBF16 = 27, kNone = -1 };

enum : int {
    kModeDequantBf16 = 0,  // grouped_matmul W8A8: int32 -> (acc*w_scale)*x_scale -> bf16
    kModeSwigluQuant = 1,  // grouped_matmul_swiglu_quant: (acc*x_scale)*w_scale -> SwiGLU -> int8 requant
    kModeInt32 = 2,        // grouped_matmul with an int32 result: raw accumulators
};

enum : int { kPathSm100 = 0, kPathSimt = 1 };

// Kernel status word (4 x int32 at the start of the workspace).  code 0 = clean.
// kStatusBadIndex: a scattered result row named a GPU that is no peer or a row outside the result; the row was skipped
// (record[1] = CTA, record[2] = 800, record[3] = the first such source row).
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadIndex = 2 };

// Per-call launch options (the internal form of gmmB200LaunchOptions, include/gmm_b200.h).  They travel with the
// problem description, so two threads launching on two streams never see each other's settings.
struct LaunchOptions {
    int max_ctas = 0;                   // cap on the CTAs of the persistent kernels, 0 = one per SM
    cudaEvent_t ev_start = nullptr;     // recorded right before / after the tensor-core kernel(s) on the launch stream
    cudaEvent_t ev_stop = nullptr;
    long long wait_limit_cycles = 0;    // bound of every device-side wait, 0 = the default (about a second)
    int test_skip_k_blocks = 0;         // test only: the TMA producer leaves out this many K blocks of its last tile, so that
                                        // the MMA issuer's bounded wait runs out (the abort path); results are undefined
};

struct Problem {
    const int8_t *x = nullptr;          // [M, K]
    const int8_t *w = nullptr;          // [E, K, N]; [E, N, K] (w_layout 1); FRACTAL_NZ [E, N/32, K/16, 16, 32] (w_layout 2)
    const void *w_scale = nullptr;      // [E, N] f32 / bf16 / f16
    int w_scale_dtype = kF32;
    const float *x_scale = nullptr;     // [M] per-token scale (may be null for mode kModeInt32)
    const void *bias = nullptr;         // [E, N] int32 or bf16, optional
    int bias_dtype = kNone;
    const int64_t *group_list = nullptr;
    int gl_len = 0;
    int gl_type = 0;                    // 0 = running total, 1 = per-group count
    int64_t M = 0, K = 0, N = 0, E = 0;
    int w_layout = 0;                   // 0 row major, 1 transposed view, 2 FRACTAL_NZ
    int64_t rows_per_group_hint = 0;    // > 0: the caller's expected rows per group (tuningConfig), else M / len(group_list) is used
    int act_type = 0;                   // GMMActType: 0 none, 1 relu, 2 gelu (tanh form), 4 fast gelu, 5 silu
    int out_f16 = 0;                    // mode kModeDequantBf16 with a float16 instead of a bfloat16 result
    int mode = kModeDequantBf16;
    void *out0 = nullptr;               // y (bf16 / int32) or q (int8 [M, N/2])
    void *out1 = nullptr;               // q_scale f32 [M] (swiglu only)
    const int64_t *out_row_index = nullptr;  // optional [M]: result row r goes to row out_row_index[r] (grouped_matmul only)
    void *out_peers[8] = {nullptr};          // with num_peers > 0: out_row_index = (gpu << 40) | row, one result buffer per gpu
    int num_peers = 0;
    // grouped_matmul_finalize_routing (mode kModeDequantBf16 with combine = 1): out0 is fp32 [out_rows, N]; row r of the
    // GEMM, weighted by logit[r], is added to (scatter_add = 1) or stored at (0) row row_index[r].
    int combine = 0;
    const float *logit = nullptr;       // [M], optional
    const void *row_index = nullptr;    // [M] int64 or int32
    int row_index_i32 = 0;
    int scatter_add = 0;
    int64_t out_rows = 0;
    const void *shared_input = nullptr; // bf16 [shared_rows, N], optional: rows [shared_offset, +shared_rows) start as
    int64_t shared_rows = 0;            // float(shared_input) * shared_weight, every other row as 0 (scatter_add only)
    int64_t shared_offset = 0;
    float shared_weight = 1.0f;
    LaunchOptions opt;
};

struct Plan {
    int path = kPathSimt;
    int num_sms = 0;
    int ctas = 1;                       // 1 = one CTA per 128-row tile, 2 = CTA pairs on 256-row tiles
    bool hybrid = false;                // with ctas == 2: a second launch with 128-row tiles takes trailing blocks of <= 128 rows
    size_t ws_bytes = 0;
    size_t off_status = 0, off_amax = 0, off_stage = 0, off_done = 0;
    size_t off_wave = 0;                // 0 = no pacing counters in this workspace
    size_t zero_bytes = 0;              // leading bytes of the workspace cleared at launch
    bool maps_ready = false;
    alignas(64) CUtensorMap map_x;
    alignas(64) CUtensorMap map_w;
};

// MoeInitRoutingV3 (moe_init_routing.cu): rows of x grouped by expert, optionally quantised per row.
struct InitRoutingProblem {
    const void *x = nullptr;            // [n, h] f32 / f16 / bf16 (int8 only without quantisation)
    int x_dtype = kBF16;
    const int *expert_idx = nullptr;    // [n, k] int32
    const float *scale = nullptr;       // quant: [expert_end - expert_start, h] smooth scale; else [n]; optional
    int64_t n = 0, k = 0, h = 0;
    int64_t expert_num = 0, expert_start = 0, expert_end = 0;
    int quant = 0;                      // 1: dynamic per-row int8 quantisation, 0: rows copied as they are
    int row_idx_type = 0;               // 0: expanded_row_idx[pair] = output row (-1 if filtered out), 1: [output row] = pair
    int count_type = 1;                 // 1: counts per active expert, 2: (expert, count) pairs of the non-empty ones
    void *expanded_x = nullptr;         // [n*k, h]
    int *expanded_row_idx = nullptr;    // [n*k]
    long long *counts_out = nullptr;    // [range] or [expert_num, 2]
    float *expanded_scale = nullptr;    // [n*k]
};
size_t init_routing_workspace_bytes(const InitRoutingProblem &r);
cudaError_t init_routing_launch(const InitRoutingProblem &r, void *workspace, size_t workspace_bytes, cudaStream_t stream);

// A non-contiguous tensor view whose contiguous copy lives in the workspace (view_copy.cu).
struct StagedView {
    std::vector<int64_t> dims, strides;  // strides in elements
    int elem = 1;                        // bytes per element
    void *data = nullptr;                // address of the view's first element
    size_t ws_off = 0;                   // offset of the contiguous copy behind the operator's own workspace
    bool is_output = false;              // outputs are copied in before and back after the operator
    void **field = nullptr;              // the pointer of the problem description that must name the copy
};
cudaError_t view_copy_launch(const StagedView &v, void *contiguous, bool to_contiguous, cudaStream_t stream);

// Host only: choose the kernel path and the workspace layout from the shapes.  Never touches the device (the tile-shape
// heuristics assume the 148 SMs of a B200; the launch itself asks the device).
void make_plan(const Problem &p, Plan *plan);
// Enqueue the operator on `stream`.  Returns cudaSuccess or the first CUDA error.
cudaError_t launch(const Problem &p, Plan &plan, void *workspace, size_t workspace_bytes, cudaStream_t stream);

// gmm_sm100.cu
bool sm100_shape_ok(const Problem &p);
cudaError_t sm100_encode_maps(const Problem &p, Plan &plan);
cudaError_t sm100_launch(const Problem &p, Plan &plan, void *workspace, cudaStream_t stream);
// gmm_simt.cu
// Initial contents of the combined result (PreProcess of grouped_matmul_finalize_routing.h:208-258).
cudaError_t combine_init_launch(const Problem &p, cudaStream_t stream);
cudaError_t simt_launch(const Problem &p, Plan &plan, void *workspace, cudaStream_t stream);

// SMs of the current device (cached per device); 0 on error.
int device_sm_count();

#ifdef __CUDACC__
// Activations of the dequantising epilogue (ActivationCompute, gmm/grouped_matmul/op_kernel/grouped_matmul_quant_mixcore.h:390-405).
// The reference calls its vector library's Relu / Gelu / FasterGelu / Silu; the library's published definitions are
//   Gelu(x)       = x / (1 + exp(-1.59576912 * (x + 0.044715 * x^3)))      (tanh form)
//   FasterGelu(x) = x / (1 + exp(-1.702 * x))
//   Silu(x)       = x / (1 + exp(-x))
// evaluated here in fp32 with every operation rounded separately.
__device__ __forceinline__ float apply_activation(int act_type, float v)
{
    switch (act_type) {
        case 1: return v > 0.0f ? v : 0.0f;
        case 2: {
            const float v3 = __fmul_rn(__fmul_rn(v, v), v);
            const float u = __fmul_rn(-1.59576912f, __fadd_rn(v, __fmul_rn(0.044715f, v3)));
            return __fdiv_rn(v, __fadd_rn(1.0f, expf(u)));
        }
        case 4: return __fdiv_rn(v, __fadd_rn(1.0f, expf(__fmul_rn(-1.702f, v))));
        case 5: return __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
        default: return v;
    }
}
#endif

}  // namespace gmm
