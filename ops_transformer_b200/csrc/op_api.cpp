// Host side of the two operators: the aclnn two-phase entry points (parameter validation, executor
// construction, launch) and the flat entry points declared in include/gmm_b200.h.
//
// Validation order and status codes follow the reference's op_api layer:
//   gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul.cpp
//       CheckNotNull :303-311, CheckCommonParam :1883-1916, CheckUnusedParams :1373-1386,
//       CheckFunctionQuantParams :786-812, CheckGroupedMatmulQuant :678-700, CheckQuantParamsDtype :642-676,
//       CheckPerTokenScale :556-588, SplitMSingleXSingleWeightSingleY :1021-1053, CheckGroupListCommonTensor :339-361
//   gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant.cpp
//       CheckNotNull :75-105, CheckInputOutDims_A8W8 :108-125, CheckInputOutShape_A8W8 :149-213, CheckDtypeValid :304-324
// restricted to the int8 x int8 path.  The first phase is host only and never reads group_list; the second
// phase enqueues on the caller's CUDA stream and returns.
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "acl_shim.h"
#include "aclnnop/aclnn_grouped_matmul_finalize_routing_weight_nz.h"
#include "aclnnop/aclnn_grouped_matmul_swiglu_quant.h"
#include "aclnnop/aclnn_grouped_matmul_swiglu_quant_weight_nz.h"
#include "aclnnop/aclnn_grouped_matmul_v4.h"
#include "aclnnop/aclnn_grouped_matmul_v5.h"
#include "aclnnop/aclnn_grouped_matmul_weight_nz.h"
#include "aclnnop/aclnn_moe_init_routing_v3.h"
#include "gmm_b200.h"

namespace gmm {
void register_executor(aclOpExecutor *e);
bool claim_executor(aclOpExecutor *e);
bool executor_is_live(aclOpExecutor *e);

namespace {

constexpr int64_t kMaxGroupListLen = 1024;   // MAX_GROUP_LIST_SIZE_TENSOR, aclnn_grouped_matmul.cpp:52
constexpr int64_t kMaxInnerAxis = 65535;     // aclnn_grouped_matmul.cpp:53
constexpr int64_t kSwigluNLimit = 10240;     // N_LIMIT, aclnn_grouped_matmul_swiglu_quant.cpp:39
constexpr int64_t kSwigluKLimit = 65536;     // K_LIMIT_A8W8, :37

#define GMM_REQUIRE(cond, code, ...)                   \
    do {                                               \
        if (!(cond)) return fail((code), __VA_ARGS__); \
    } while (0)

bool is_private_format(aclFormat f) { return f == ACL_FORMAT_FRACTAL_NZ || f == ACL_FORMAT_FRACTAL_Z || f == ACL_FORMAT_NC1HWC0; }

// Same test as IsTransposeLastTwoDims (gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_util.cpp:16-33).
bool is_transposed_last_two(const aclTensor *t)
{
    const size_t r = t->rank();
    if (r < 2) return false;
    const size_t d1 = r - 1, d2 = r - 2;
    if (t->strides[d2] == 1 && t->strides[d1] == t->dim(d2)) {
        int64_t acc = t->dim(d1) * t->dim(d2);
        for (size_t b = r - 2; b-- > 0;) {
            if (t->strides[b] != acc) return false;
            acc *= t->dim(b);
        }
        return true;
    }
    return false;
}

aclOpExecutor *new_executor(const char *name)
{
    aclOpExecutor *e = new (std::nothrow) aclOpExecutor();
    if (e) e->op_name = name;
    return e;
}

// Address the operator will use for tensor `t`: the tensor's own memory when it is contiguous; otherwise a contiguous
// copy in the workspace tail, filled before the launch (and, for an output, copied back afterwards).  The address of a
// copy is only known in the second phase: until then `*field` holds an aligned stand-in.
template <typename P>
void bind_tensor(aclOpExecutor *e, const aclTensor *t, P *field, bool is_output, bool contiguous_enough = false)
{
    if (!t) { *field = nullptr; return; }
    if (t->contiguous() || contiguous_enough) { *field = (P)tensor_ptr(t); return; }
    StagedView v;
    v.dims = t->view_dims;
    v.strides = t->strides;
    v.elem = (int)dtype_size(t->dtype);
    v.data = tensor_ptr(t);
    v.ws_off = e->staged_bytes;
    v.is_output = is_output;
    v.field = (void **)field;  // the field is a pointer of some type; only its value is replaced
    e->staged_bytes += ((size_t)t->numel() * v.elem + 255) / 256 * 256;
    e->staged.push_back(v);
    *field = (P)(uintptr_t)4096;
}

// Env-gated profiler ranges around both phases of every entry point (GMM_B200_NVTX=1), the counterpart of the
// reference's L2_DFX_PHASE_1 / L2_DFX_PHASE_2 (gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul.cpp:2005, 2151).
// NVTX is header only and does nothing unless a tool is attached.
bool nvtx_enabled()
{
    static const bool on = [] {
        const char *e = std::getenv("GMM_B200_NVTX");
        return e && e[0] && e[0] != '0';
    }();
    return on;
}
struct PhaseRange {
    bool on;
    PhaseRange(const char *op, int phase) : on(nvtx_enabled())
    {
        if (!on) return;
        char name[160];
        std::snprintf(name, sizeof(name), "%s phase %d", op, phase);
        nvtxRangePushA(name);
    }
    ~PhaseRange()
    {
        if (on) nvtxRangePop();
    }
};

// Public options -> internal form.  Fields beyond the caller's structSize read as zero.
aclnnStatus convert_options(const gmmB200LaunchOptions *o, LaunchOptions *out)
{
    *out = LaunchOptions();
    if (!o) return ACLNN_SUCCESS;
    gmmB200LaunchOptions full;
    std::memset(&full, 0, sizeof(full));
    const size_t n = o->structSize < sizeof(full) ? o->structSize : sizeof(full);
    GMM_REQUIRE(n >= 8, ACLNN_ERR_PARAM_INVALID, "gmmB200LaunchOptions.structSize %u is too small.", o->structSize);
    std::memcpy(&full, o, n);
    GMM_REQUIRE(full.maxCtas >= 0 && full.waitLimitCycles >= 0 && full.testSkipKBlocks >= 0, ACLNN_ERR_PARAM_INVALID,
                "gmmB200LaunchOptions: maxCtas, waitLimitCycles and testSkipKBlocks must not be negative.");
    GMM_REQUIRE((full.startEvent == nullptr) == (full.stopEvent == nullptr), ACLNN_ERR_PARAM_INVALID,
                "gmmB200LaunchOptions: startEvent and stopEvent come together or not at all.");
    out->max_ctas = full.maxCtas;
    out->ev_start = static_cast<cudaEvent_t>(full.startEvent);
    out->ev_stop = static_cast<cudaEvent_t>(full.stopEvent);
    out->wait_limit_cycles = full.waitLimitCycles;
    out->test_skip_k_blocks = full.testSkipKBlocks;
    return ACLNN_SUCCESS;
}

aclnnStatus finish_phase1(aclOpExecutor *e, uint64_t *workspaceSize, aclOpExecutor **executor)
{
    // kInitRouting stores its size in plan.ws_bytes too
    *workspaceSize = e->kind == aclOpExecutor::kNoop ? 0 : e->plan.ws_bytes + e->staged_bytes;
    register_executor(e);
    *executor = e;
    return ACLNN_SUCCESS;
}

}  // namespace

aclnnStatus run_executor(const char *op_name, void *workspace, uint64_t workspace_size, aclOpExecutor *executor,
                         aclrtStream stream)
{
    clear_error();
    PhaseRange phase_range(op_name, 2);
    GMM_REQUIRE(executor != nullptr, ACLNN_ERR_PARAM_NULLPTR, "%s: executor must not be nullptr.", op_name);
    GMM_REQUIRE(claim_executor(executor), ACLNN_ERR_PARAM_INVALID,
                "%s: executor is not live; an executor can be run once and only after its GetWorkspaceSize call.", op_name);
    aclnnStatus rc = ACLNN_SUCCESS;
    if (std::strcmp(executor->op_name, op_name) != 0) {
        rc = fail(ACLNN_ERR_PARAM_INVALID, "%s: executor was built by %s.", op_name, executor->op_name);
    } else if (executor->kind != aclOpExecutor::kNoop) {
        const size_t need = executor->plan.ws_bytes + executor->staged_bytes;
        if (workspace_size < need) {
            rc = fail(ACLNN_ERR_PARAM_INVALID, "%s: workspaceSize %llu is smaller than the %llu bytes required.", op_name,
                      (unsigned long long)workspace_size, (unsigned long long)need);
        } else if (need && !workspace) {
            rc = fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspace must not be nullptr.", op_name);
        } else {
            cudaStream_t cs = static_cast<cudaStream_t>(stream);
            char *tail = static_cast<char *>(workspace) + executor->plan.ws_bytes;
            cudaError_t ce = cudaSuccess;
            for (StagedView &v : executor->staged) {  // contiguous copies of the strided views (outputs too: rows the
                *v.field = tail + v.ws_off;           // operator leaves alone must keep their contents)
                if (ce == cudaSuccess) ce = view_copy_launch(v, tail + v.ws_off, true, cs);
            }
            if (executor->kind == aclOpExecutor::kGmm && executor->plan.path == kPathSm100 && !sm100_shape_ok(executor->problem))
                executor->plan.path = kPathSimt;      // a workspace that is not 16-byte aligned cannot feed TMA
            if (ce == cudaSuccess)
                ce = executor->kind == aclOpExecutor::kInitRouting
                         ? init_routing_launch(executor->routing, workspace, executor->plan.ws_bytes, cs)
                         : launch(executor->problem, executor->plan, workspace, executor->plan.ws_bytes, cs);
            for (StagedView &v : executor->staged)
                if (v.is_output && ce == cudaSuccess) ce = view_copy_launch(v, tail + v.ws_off, false, cs);
            if (ce != cudaSuccess)
                rc = fail(ACLNN_ERR_INNER, "%s: kernel launch failed: %s", op_name, cudaGetErrorString(ce));
        }
    }
    delete executor;
    return rc;
}

}  // namespace gmm

using namespace gmm;

extern "C" {

int32_t gmmB200Version(void) { return 100; }

aclnnStatus gmmB200SetExecutorOptions(aclOpExecutor *executor, const gmmB200LaunchOptions *options)
{
    clear_error();
    GMM_REQUIRE(executor != nullptr, ACLNN_ERR_PARAM_NULLPTR, "executor must not be nullptr.");
    GMM_REQUIRE(executor_is_live(executor), ACLNN_ERR_PARAM_INVALID,
                "executor is not live; options are set between GetWorkspaceSize and the second-phase call.");
    return convert_options(options, &executor->problem.opt);
}

// Shared first phase of aclnnGroupedMatmulV4 / V5 / WeightNz (aclnnGroupedMatmulGetWorkspaceSizeCommon,
// gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul.cpp:1839-1880).  force_nz: the weight's storage is FRACTAL_NZ
// whatever its format field says (the WeightNz entry point, :1917-1955).
static aclnnStatus gmm_phase1(const char *kOp, bool force_nz, int64_t rows_hint,
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclTensorList *out, aclTensorList *activationFeatureOutOptional,
    aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize, aclOpExecutor **executor)
{
    clear_error();
    // CheckNotNull
    GMM_REQUIRE(x != nullptr, ACLNN_ERR_PARAM_NULLPTR, "x must not be nullptr.");
    GMM_REQUIRE(!x->items.empty(), ACLNN_ERR_PARAM_INVALID, "x must not be empty tensorlist.");
    (void)kOp;
    GMM_REQUIRE(weight != nullptr, ACLNN_ERR_PARAM_NULLPTR, "weight must not be nullptr.");
    GMM_REQUIRE(!weight->items.empty(), ACLNN_ERR_PARAM_INVALID, "weight must not be empty tensorlist.");
    GMM_REQUIRE(out != nullptr, ACLNN_ERR_PARAM_NULLPTR, "y must not be nullptr.");
    GMM_REQUIRE(!out->items.empty(), ACLNN_ERR_PARAM_INVALID, "y must not be empty tensorlist.");
    GMM_REQUIRE(workspaceSize != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspaceSize must not be nullptr.");
    GMM_REQUIRE(executor != nullptr, ACLNN_ERR_PARAM_NULLPTR, "executor must not be nullptr.");

    // CheckCommonParam
    GMM_REQUIRE(groupType != 1, ACLNN_ERR_PARAM_INVALID, "Not support split n dim now, groupType can not be 1.");
    GMM_REQUIRE(groupType == 0 || groupType == 2 || groupType == -1, ACLNN_ERR_PARAM_INVALID,
                "groupType only support -1/0/2 now, but given groupType is %lld", (long long)groupType);
    if (splitItem == 2 || splitItem == 3)
        GMM_REQUIRE(groupType != -1, ACLNN_ERR_PARAM_INVALID, "When splitItem is 2/3, groupType can not be -1.");
    GMM_REQUIRE(groupListOptional == nullptr || groupListOptional->rank() == (groupListType == 2 ? 2u : 1u),
                ACLNN_ERR_PARAM_INVALID, "groupList dim only support 1 (2 only when groupListType is 2), but now is %zu.",
                groupListOptional->rank());
    GMM_REQUIRE(actType >= 0, ACLNN_ERR_PARAM_INVALID, "actType must be larger or equal to 0");
    GMM_REQUIRE(actType != GMM_ACT_TYPE_GELU_ERR_FUNC, ACLNN_ERR_PARAM_INVALID, "Activation function not support GELU_ERR_FUNC now.");
    GMM_REQUIRE(actType <= GMM_ACT_TYPE_SILU, ACLNN_ERR_PARAM_INVALID, "Activation function only support RELU/GELU_TANH/FASTGELU/SILU.");
    GMM_REQUIRE(groupListType == 0 || groupListType == 1, ACLNN_ERR_PARAM_INVALID,
                "groupListType should be 0 or 1 (the sparse type 2 is not supported on this platform).");

    // CheckUnusedParams
    GMM_REQUIRE(activationInputOptional == nullptr, ACLNN_ERR_PARAM_INVALID, "activationInputOptional must be nullptr.");
    GMM_REQUIRE(activationQuantScaleOptional == nullptr, ACLNN_ERR_PARAM_INVALID, "activationQuantScaleOptional must be nullptr.");
    GMM_REQUIRE(activationQuantOffsetOptional == nullptr, ACLNN_ERR_PARAM_INVALID, "activationQuantOffsetOptional must be nullptr.");
    GMM_REQUIRE(activationFeatureOutOptional == nullptr, ACLNN_ERR_PARAM_INVALID, "activationFeatureOutOptional must be nullptr.");
    GMM_REQUIRE(dynQuantScaleOutOptional == nullptr, ACLNN_ERR_PARAM_INVALID, "dynQuantScaleOutOptional must be nullptr.");

    // Scope of this build: one x, one weight, one y, rows split along M.
    GMM_REQUIRE(groupType == 0, ACLNN_ERR_PARAM_INVALID, "this build supports groupType 0 (split M) only, got %lld.", (long long)groupType);
    GMM_REQUIRE(x->items.size() == 1 && weight->items.size() == 1 && out->items.size() == 1, ACLNN_ERR_PARAM_INVALID,
                "this build supports single-tensor x, weight and y only (sizes %zu, %zu, %zu).", x->items.size(),
                weight->items.size(), out->items.size());
    GMM_REQUIRE(splitItem == 2 || splitItem == 3, ACLNN_ERR_PARAM_INVALID,
                "When y is not separated, splitItem should be 2/3, but current splitItem is %lld.", (long long)splitItem);
    const aclTensor *tx = x->items[0], *tw = weight->items[0], *ty = out->items[0];
    GMM_REQUIRE(tx && tw && ty, ACLNN_ERR_PARAM_INVALID, "x[0], weight[0] and y[0] must not be null.");

    // CheckFunctionParams: the int8 x int8 family.
    GMM_REQUIRE(tx->dtype == ACL_INT8 && tw->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID,
                "this build supports int8 x with int8 weight only.");
    GMM_REQUIRE(ty->dtype == ACL_BF16 || ty->dtype == ACL_FLOAT16 || ty->dtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID,
                "Expect yDtype is int32, float16 or bfloat16 in quant case on this build (the int8 result is not implemented).");
    const aclTensor *tbias = nullptr;
    if (biasOptional != nullptr && !biasOptional->items.empty()) {
        GMM_REQUIRE(biasOptional->items.size() == 1 && biasOptional->items[0], ACLNN_ERR_PARAM_INVALID, "bias must hold one tensor.");
        tbias = biasOptional->items[0];
        GMM_REQUIRE(tbias->dtype == ACL_INT32 || tbias->dtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID,
                    "GMM: bias dtype does not match with required dtype int32 or bfloat16.");
    }
    const bool int32_out = ty->dtype == ACL_INT32;
    const aclTensor *tscale = nullptr, *tpts = nullptr;
    if (!int32_out) {
        // CheckGroupedMatmulQuant
        GMM_REQUIRE(offsetOptional == nullptr, ACLNN_ERR_PARAM_INVALID, "GMM: offset must be nullptr in quant, but now is not nullptr.");
        GMM_REQUIRE(scaleOptional != nullptr, ACLNN_ERR_PARAM_INVALID, "GMM: scale must not be nullptr in quant, but now is nullptr.");
        GMM_REQUIRE(scaleOptional->items.size() == 1 && scaleOptional->items[0], ACLNN_ERR_PARAM_INVALID, "Invalid scale.");
        tscale = scaleOptional->items[0];
        // Reference pairs (bf16 scale, bf16 y); fp32 scale with a bf16 result is accepted as an extension
        // (the kernel converts every scale to fp32, grouped_matmul_quant_mixcore.h:262).
        if (ty->dtype == ACL_FLOAT16)
            GMM_REQUIRE(tscale->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID,
                        "quant case only supports scale with data type float32 when output is float16.");
        else
            GMM_REQUIRE(tscale->dtype == ACL_BF16 || tscale->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID,
                        "quant case supports scale data type bfloat16 or float32 with output data type bfloat16.");
        if (perTokenScaleOptional != nullptr) {
            GMM_REQUIRE(perTokenScaleOptional->items.size() == 1, ACLNN_ERR_PARAM_INVALID,
                        "perTokenScaleOptional size[%zu] must be 1 and equal with x size[1].", perTokenScaleOptional->items.size());
            tpts = perTokenScaleOptional->items[0];
            GMM_REQUIRE(tpts != nullptr, ACLNN_ERR_PARAM_INVALID, "perTokenScaleOptional[0] must not be nullptr, but now is nullptr.");
            GMM_REQUIRE(tpts->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "per-token quant case only support perTokenScale with data type float32.");
            GMM_REQUIRE(tpts->rank() == 1, ACLNN_ERR_PARAM_INVALID,
                        "perTokenScaleOptional dim num must be 1 when x is single tensor, but now is %zu.", tpts->rank());
        }
        GMM_REQUIRE(antiquantScaleOptional == nullptr && antiquantOffsetOptional == nullptr, ACLNN_ERR_PARAM_INVALID,
                    "Detected quant, but antiquant inputs is not empty!");
    }

    // SplitMSingleXSingleWeightSingleY: dims and shapes x(m,k), weight(e,k,n), y(m,n).
    GMM_REQUIRE(!is_private_format(tx->format) && !is_private_format(ty->format), ACLNN_ERR_PARAM_INVALID, "Invalid format.");
    const bool w_nz = force_nz || tw->format == ACL_FORMAT_FRACTAL_NZ;
    GMM_REQUIRE(w_nz || !is_private_format(tw->format), ACLNN_ERR_PARAM_INVALID, "Invalid weight format.");
    GMM_REQUIRE(tx->rank() == 2, ACLNN_ERR_PARAM_INVALID, "x[0] dim num should be 2 in this case, but now is %zu.", tx->rank());
    GMM_REQUIRE(ty->rank() == 2, ACLNN_ERR_PARAM_INVALID, "y[0] dim num should be 2 in this case, but now is %zu.", ty->rank());
    const int64_t M = tx->dim(0), K = tx->dim(1), E = tw->rank() ? tw->dim(0) : 0;
    int64_t N = 0;
    if (w_nz && tw->rank() == 5) {
        // FRACTAL_NZ view [E, N/32, K/16, 16, 32] (int8 fractal 16 x 32)
        GMM_REQUIRE(tw->dim(3) == 16 && tw->dim(4) == 32 && tw->dim(2) * 16 == K, ACLNN_ERR_PARAM_INVALID,
                    "FRACTAL_NZ weight must be [E, N/32, K/16, 16, 32] with K/16 * 16 equal to x's K.");
        N = tw->dim(1) * 32;
    } else {
        GMM_REQUIRE(tw->rank() == 3, ACLNN_ERR_PARAM_INVALID, "weight[0] dim num should be 3 in this case, but now is %zu.", tw->rank());
        N = tw->dim(2);
        GMM_REQUIRE(tw->dim(1) == K, ACLNN_ERR_PARAM_INVALID, "k dim value of x and weight is not matched.");
        if (w_nz) GMM_REQUIRE(K % 16 == 0 && N % 32 == 0, ACLNN_ERR_PARAM_INVALID, "FRACTAL_NZ weight needs K %% 16 == 0 and N %% 32 == 0.");
    }
    GMM_REQUIRE(ty->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "m dim value of x and y is not matched.");
    GMM_REQUIRE(ty->dim(1) == N, ACLNN_ERR_PARAM_INVALID, "n dim value of weight and y is not matched.");
    GMM_REQUIRE(K <= kMaxInnerAxis && N <= kMaxInnerAxis, ACLNN_ERR_PARAM_INVALID, "inner axis of x / weight must not exceed %lld.", (long long)kMaxInnerAxis);
    // CheckGroupListCommonTensor
    GMM_REQUIRE(groupListOptional != nullptr, ACLNN_ERR_PARAM_INVALID, "groupListOptional(tensor) is required in this case, but get nullptr.");
    const int64_t glLen = groupListOptional->dim(0);
    GMM_REQUIRE(glLen <= kMaxGroupListLen, ACLNN_ERR_PARAM_INVALID,
                "When groupList type is tensor, size of groupList %lld should be less than or equal to %lld.", (long long)glLen, (long long)kMaxGroupListLen);
    GMM_REQUIRE((glLen == E && E > 1) || E == 1, ACLNN_ERR_PARAM_INVALID,
                "When groupList is not null, size of groupList(tensor) %lld should be equal to weight dim 0 %lld with groupType 0.", (long long)glLen, (long long)E);
    GMM_REQUIRE(groupListOptional->dtype == ACL_INT64, ACLNN_ERR_PARAM_INVALID, "Invalid dtype: Only int64 is supported for groupList.");
    if (tscale) {
        GMM_REQUIRE(tscale->rank() == 2 && tscale->dim(0) == E && tscale->dim(1) == N, ACLNN_ERR_PARAM_INVALID, "scale shape must be [%lld, %lld].", (long long)E, (long long)N);
    }
    if (tpts) {
        GMM_REQUIRE(tpts->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "MDim[%lld] of perTokenScaleOptional should be equal with MDim[%lld] of x.", (long long)tpts->dim(0), (long long)M);
    }
    if (tbias) {
        GMM_REQUIRE(tbias->rank() == 2 && tbias->dim(0) == E && tbias->dim(1) == N, ACLNN_ERR_PARAM_INVALID, "bias shape must be [%lld, %lld].", (long long)E, (long long)N);
    }

    aclOpExecutor *e = new_executor(kOp);
    GMM_REQUIRE(e != nullptr, ACLNN_ERR_INNER_CREATE_EXECUTOR, "cannot create executor.");
    // Empty tensors: nothing to launch and a workspace of 0 (CheckZeroShape, aclnn_grouped_matmul.cpp:1535-1548 with its
    // caller :1770-1772: an x without elements, i.e. M == 0 or K == 0, returns success before anything is built).
    if (M == 0 || K == 0 || N == 0 || glLen == 0) return finish_phase1(e, workspaceSize, executor);

    const bool w_trans = !w_nz && !tw->contiguous() && is_transposed_last_two(tw);
    // Strided views are served through contiguous copies in the workspace (Contiguous / ViewCopy of the reference,
    // aclnn_grouped_matmul.cpp:1640-1667, 1802-1805); the transposed weight view and the fractal storage are read as they lie.
    Problem &p = e->problem;
    bind_tensor(e, tx, &p.x, false);
    bind_tensor(e, tw, &p.w, false, w_trans || w_nz);
    bind_tensor(e, tscale, &p.w_scale, false);
    p.w_scale_dtype = tscale ? (int)tscale->dtype : kF32;
    bind_tensor(e, tpts, &p.x_scale, false);
    bind_tensor(e, tbias, &p.bias, false);
    p.bias_dtype = tbias ? (int)tbias->dtype : kNone;
    bind_tensor(e, groupListOptional, &p.group_list, false);
    p.gl_len = (int)(E == 1 ? 1 : glLen);
    p.gl_type = (int)groupListType;
    p.M = M; p.K = K; p.N = N; p.E = E;
    p.w_layout = w_nz ? 2 : (w_trans ? 1 : 0);
    p.rows_per_group_hint = rows_hint;
    // The reference's test for an activation with an int32 result never fires (aclnn_grouped_matmul.cpp:984-985) and its
    // int32 kernel has no vector stage: the activation is accepted and has no effect.
    p.act_type = int32_out ? 0 : (int)actType;
    p.mode = int32_out ? kModeInt32 : kModeDequantBf16;
    p.out_f16 = ty->dtype == ACL_FLOAT16 ? 1 : 0;
    bind_tensor(e, ty, &p.out0, true);
    e->kind = aclOpExecutor::kGmm;
    make_plan(p, &e->plan);
    return finish_phase1(e, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulV4GetWorkspaceSize(
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclTensorList *out, aclTensorList *activationFeatureOutOptional,
    aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize, aclOpExecutor **executor)
{
    return gmm_phase1("aclnnGroupedMatmulV4", false, 0, x, weight, biasOptional, scaleOptional, offsetOptional, antiquantScaleOptional,
                      antiquantOffsetOptional, perTokenScaleOptional, groupListOptional, activationInputOptional,
                      activationQuantScaleOptional, activationQuantOffsetOptional, splitItem, groupType, groupListType, actType, out,
                      activationFeatureOutOptional, dynQuantScaleOutOptional, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulV4(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulV4", workspace, workspaceSize, executor, stream);
}

// tuningConfigOptional[0] is the number of rows the caller expects per group, a hint for the reference's host tiling
// (aclnn_grouped_matmul.cpp:1336-1360).  The device scheduler here reads group_list itself; the hint only replaces
// M / len(group_list) in the choice between 128-row tiles and CTA pairs, which matters when many groups are empty.
static aclnnStatus check_tuning_config(const aclIntArray *cfg, int64_t *rows_hint)
{
    *rows_hint = 0;
    if (cfg) {
        for (int64_t v : cfg->values)
            if (v < 0) return fail(ACLNN_ERR_PARAM_INVALID, "tuningConfig values must not be negative.");
        if (!cfg->values.empty()) *rows_hint = cfg->values[0];
    }
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnGroupedMatmulV5GetWorkspaceSize(
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclIntArray *tuningConfigOptional, aclTensorList *out, aclTensorList *activationFeatureOutOptional,
    aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize, aclOpExecutor **executor)
{
    clear_error();
    int64_t rows_hint = 0;
    if (check_tuning_config(tuningConfigOptional, &rows_hint) != ACLNN_SUCCESS) return ACLNN_ERR_PARAM_INVALID;
    return gmm_phase1("aclnnGroupedMatmulV5", false, rows_hint, x, weight, biasOptional, scaleOptional, offsetOptional, antiquantScaleOptional,
                      antiquantOffsetOptional, perTokenScaleOptional, groupListOptional, activationInputOptional,
                      activationQuantScaleOptional, activationQuantOffsetOptional, splitItem, groupType, groupListType, actType, out,
                      activationFeatureOutOptional, dynQuantScaleOutOptional, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulV5(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulV5", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnGroupedMatmulWeightNzGetWorkspaceSize(
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclIntArray *tuningConfigOptional, int64_t quantGroupSize, aclTensorList *out,
    aclTensorList *activationFeatureOutOptional, aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize,
    aclOpExecutor **executor)
{
    clear_error();
    int64_t rows_hint = 0;
    if (check_tuning_config(tuningConfigOptional, &rows_hint) != ACLNN_SUCCESS) return ACLNN_ERR_PARAM_INVALID;
    GMM_REQUIRE(quantGroupSize >= 0, ACLNN_ERR_PARAM_INVALID, "quantGroupSize must not be negative.");
    return gmm_phase1("aclnnGroupedMatmulWeightNz", true, rows_hint, x, weight, biasOptional, scaleOptional, offsetOptional,
                      antiquantScaleOptional, antiquantOffsetOptional, perTokenScaleOptional, groupListOptional,
                      activationInputOptional, activationQuantScaleOptional, activationQuantOffsetOptional, splitItem, groupType,
                      groupListType, actType, out, activationFeatureOutOptional, dynQuantScaleOutOptional, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulWeightNz(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulWeightNz", workspace, workspaceSize, executor, stream);
}

// ------------------------------------------------------------------------------------------------------------
// MoeInitRoutingV3
// ------------------------------------------------------------------------------------------------------------

// Checks of CheckParams (moe/moe_init_routing_v3/op_host/op_api/aclnn_moe_init_routing_v3.cpp:52-181) in their order, then the
// attribute rules the reference enforces in its tiling (README.md "constraints"): dropPadMode 0, expertTokensNumType 1 or 2,
// expertTokensNumFlag true, quantMode 1 or -1, rowIdxType 0 or 1, activeNum = n*k (or 0), 0 <= start < end <= expertNum.
aclnnStatus aclnnMoeInitRoutingV3GetWorkspaceSize(const aclTensor *x, const aclTensor *expertIdx, const aclTensor *scaleOptional,
                                                  const aclTensor *offsetOptional, int64_t activeNum, int64_t expertCapacity,
                                                  int64_t expertNum, int64_t dropPadMode, int64_t expertTokensNumType,
                                                  bool expertTokensNumFlag, int64_t quantMode,
                                                  const aclIntArray *activeExpertRangeOptional, int64_t rowIdxType,
                                                  const aclTensor *expandedXOut, const aclTensor *expandedRowIdxOut,
                                                  const aclTensor *expertTokensCountOrCumsumOut, const aclTensor *expandedScaleOut,
                                                  uint64_t *workspaceSize, aclOpExecutor **executor)
{
    static const char *kOp = "aclnnMoeInitRoutingV3";
    clear_error();
    PhaseRange phase_range(kOp, 1);
    GMM_REQUIRE(workspaceSize != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspaceSize must not be nullptr.");
    GMM_REQUIRE(executor != nullptr, ACLNN_ERR_PARAM_NULLPTR, "executor must not be nullptr.");
    GMM_REQUIRE(x && expertIdx && expandedXOut && expandedRowIdxOut && expertTokensCountOrCumsumOut && expandedScaleOut,
                ACLNN_ERR_PARAM_NULLPTR, "x, expertIdx and the four outputs must not be nullptr.");
    GMM_REQUIRE(x->dtype == ACL_FLOAT16 || x->dtype == ACL_BF16 || x->dtype == ACL_FLOAT || x->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID,
                "x dtype must be float16, bfloat16, float32 or int8.");
    GMM_REQUIRE(expertIdx->dtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID, "expertIdx dtype must be int32.");
    GMM_REQUIRE(!scaleOptional || scaleOptional->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "scale dtype must be float32.");
    GMM_REQUIRE(!offsetOptional || offsetOptional->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "offset dtype must be float32.");
    GMM_REQUIRE(expandedXOut->dtype == ACL_FLOAT16 || expandedXOut->dtype == ACL_BF16 || expandedXOut->dtype == ACL_FLOAT ||
                    expandedXOut->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID, "expandedXOut dtype must be float16, bfloat16, float32 or int8.");
    GMM_REQUIRE(expandedRowIdxOut->dtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID, "expandedRowIdxOut dtype must be int32.");
    GMM_REQUIRE(expertTokensCountOrCumsumOut->dtype == ACL_INT64, ACLNN_ERR_PARAM_INVALID, "expertTokensCountOrCumsumOut dtype must be int64.");
    GMM_REQUIRE(expandedScaleOut->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "expandedScaleOut dtype must be float32.");
    // the reference dereferences the range without a test (:100); a missing range is refused here
    GMM_REQUIRE(activeExpertRangeOptional && activeExpertRangeOptional->values.size() == 2, ACLNN_ERR_PARAM_INVALID,
                "activeExpertRange must hold [expertStart, expertEnd].");
    const int64_t eStart = activeExpertRangeOptional->values[0], eEnd = activeExpertRangeOptional->values[1];
    const int64_t range = eEnd - eStart;
    GMM_REQUIRE(x->rank() == 2 && expertIdx->rank() == 2, ACLNN_ERR_PARAM_INVALID, "x and expertIdx must have 2 dimensions.");
    const int64_t n = x->dim(0), h = x->dim(1), k = expertIdx->dim(1);
    GMM_REQUIRE(expertIdx->dim(0) == n, ACLNN_ERR_PARAM_INVALID, "expertIdx shape error");
    if (scaleOptional && quantMode != 0) {
        if (quantMode == -1)
            GMM_REQUIRE(scaleOptional->rank() == 1 && scaleOptional->dim(0) == n, ACLNN_ERR_PARAM_INVALID, "scale shape error");
        else if (quantMode == 1)
            GMM_REQUIRE(scaleOptional->rank() == 2 && scaleOptional->dim(0) == range && scaleOptional->dim(1) == h, ACLNN_ERR_PARAM_INVALID,
                        "scale shape error");
        GMM_REQUIRE(expandedScaleOut->rank() == 1 && expandedScaleOut->dim(0) == n * k, ACLNN_ERR_PARAM_INVALID, "expandedScaleOut shape error");
    }
    GMM_REQUIRE(expandedXOut->rank() == 2 && expandedXOut->dim(0) == n * k && expandedXOut->dim(1) == h, ACLNN_ERR_PARAM_INVALID,
                "expandedXOut shape error");
    GMM_REQUIRE(expandedRowIdxOut->rank() == 1 && expandedRowIdxOut->dim(0) == n * k, ACLNN_ERR_PARAM_INVALID, "expandedRowIdxOut shape error");
    if (expertTokensNumType == 1)
        GMM_REQUIRE(expertTokensCountOrCumsumOut->rank() == 1 && expertTokensCountOrCumsumOut->dim(0) == range, ACLNN_ERR_PARAM_INVALID,
                    "expertTokensCountOrCumsumOut shape error");
    else if (expertTokensNumType == 2)
        GMM_REQUIRE(expertTokensCountOrCumsumOut->rank() == 2 && expertTokensCountOrCumsumOut->dim(0) == expertNum &&
                        expertTokensCountOrCumsumOut->dim(1) == 2, ACLNN_ERR_PARAM_INVALID, "expertTokensCountOrCumsumOut shape error");
    // attributes
    GMM_REQUIRE(dropPadMode == 0, ACLNN_ERR_PARAM_INVALID, "dropPadMode only supports 0 (dropless).");
    GMM_REQUIRE(expertTokensNumType == 1 || expertTokensNumType == 2, ACLNN_ERR_PARAM_INVALID, "expertTokensNumType only supports 1 (count) and 2 (key_value).");
    GMM_REQUIRE(expertTokensNumFlag, ACLNN_ERR_PARAM_INVALID, "expertTokensNumFlag only supports true.");
    GMM_REQUIRE(quantMode == 1 || quantMode == -1, ACLNN_ERR_PARAM_INVALID, "quantMode only supports 1 (dynamic quant) and -1 (no quant).");
    GMM_REQUIRE(rowIdxType == 0 || rowIdxType == 1, ACLNN_ERR_PARAM_INVALID, "rowIdxType only supports 0 (gather) and 1 (scatter).");
    GMM_REQUIRE(expertCapacity >= 0, ACLNN_ERR_PARAM_INVALID, "expertCapacity must not be negative.");
    GMM_REQUIRE(activeNum == 0 || activeNum == n * k, ACLNN_ERR_PARAM_INVALID, "activeNum must equal NUM_ROWS * K.");
    GMM_REQUIRE(expertNum > 0 && expertNum <= (expertTokensNumType == 2 ? 5120 : 10240), ACLNN_ERR_PARAM_INVALID, "expertNum out of range.");
    GMM_REQUIRE(eStart >= 0 && eStart < eEnd && eEnd <= expertNum, ACLNN_ERR_PARAM_INVALID, "activeExpertRange must satisfy 0 <= start < end <= expertNum.");
    GMM_REQUIRE(n * k <= 0x7fffffffll && h <= 0x7fffffffll, ACLNN_ERR_PARAM_INVALID, "too many rows.");
    if (quantMode == 1) {
        GMM_REQUIRE(x->dtype != ACL_INT8, ACLNN_ERR_PARAM_INVALID, "dynamic quant needs a floating-point x.");
        GMM_REQUIRE(expandedXOut->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID, "dynamic quant writes an int8 expandedXOut.");
    } else {
        GMM_REQUIRE(expandedXOut->dtype == x->dtype, ACLNN_ERR_PARAM_INVALID, "without quantisation expandedXOut has x's dtype.");
    }
    aclOpExecutor *e = new_executor(kOp);
    GMM_REQUIRE(e != nullptr, ACLNN_ERR_INNER_CREATE_EXECUTOR, "cannot create executor.");
    if (n * k == 0 || h == 0) return finish_phase1(e, workspaceSize, executor);
    InitRoutingProblem &r = e->routing;
    bind_tensor(e, x, &r.x, false);
    r.x_dtype = (int)x->dtype;
    bind_tensor(e, expertIdx, &r.expert_idx, false);
    bind_tensor(e, scaleOptional, &r.scale, false);
    r.n = n; r.k = k; r.h = h;
    r.expert_num = expertNum; r.expert_start = eStart; r.expert_end = eEnd;
    r.quant = quantMode == 1;
    r.row_idx_type = (int)rowIdxType;
    r.count_type = (int)expertTokensNumType;
    bind_tensor(e, expandedXOut, &r.expanded_x, true);
    bind_tensor(e, expandedRowIdxOut, &r.expanded_row_idx, true);
    bind_tensor(e, expertTokensCountOrCumsumOut, &r.counts_out, true);
    bind_tensor(e, expandedScaleOut, &r.expanded_scale, true);
    e->kind = aclOpExecutor::kInitRouting;
    e->plan.ws_bytes = init_routing_workspace_bytes(r);
    return finish_phase1(e, workspaceSize, executor);
}

aclnnStatus aclnnMoeInitRoutingV3(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream)
{
    return run_executor("aclnnMoeInitRoutingV3", workspace, workspaceSize, executor, stream);
}

// ------------------------------------------------------------------------------------------------------------
// grouped_matmul_finalize_routing, W8A8 with a FRACTAL_NZ weight
// ------------------------------------------------------------------------------------------------------------

// Shared first phase of aclnnGroupedMatmulFinalizeRoutingWeightNz and its V2 twin.  Checks in the reference's order:
// CheckSupportScene (aclnn_grouped_matmul_finalize_routing.cpp:913-946), PreMatmulCalcProcess (:775-789), CheckParams
// (:617-636: CheckDtypeValid :252-307, CheckShape :531-588, CheckFormat :319-339, CheckEmptyTensor, CheckTuningConfig).
static aclnnStatus finalize_routing_phase1(const char *kOp, const aclTensor *x1, const aclTensor *x2, const aclTensor *scale,
                                           const aclTensor *bias, const aclTensor *offset, const aclTensor *pertokenScale,
                                           const aclTensor *groupList, const aclTensor *sharedInput, const aclTensor *logit,
                                           const aclTensor *rowIndex, int64_t dtype, float sharedInputWeight,
                                           int64_t sharedInputOffset, bool transposeX1, bool transposeX2, int64_t groupListType,
                                           const aclIntArray *tuningConfig, aclTensor *out, uint64_t *workspaceSize,
                                           aclOpExecutor **executor)
{
    clear_error();
    PhaseRange phase_range(kOp, 1);
    GMM_REQUIRE(workspaceSize != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspaceSize must not be nullptr.");
    GMM_REQUIRE(executor != nullptr, ACLNN_ERR_PARAM_NULLPTR, "executor must not be nullptr.");
    // Two supported scenes: shared input, logit and row index all given (rows are added), or row index alone (rows are stored).
    const bool base = x1 && x2 && scale && groupList && rowIndex;
    GMM_REQUIRE(base && ((sharedInput && logit) || (!sharedInput && !logit)), ACLNN_ERR_PARAM_NULLPTR,
                "GroupedMatmulFinalizeRoutingWeightNz do not support input nullptr.");
    GMM_REQUIRE(dtype == 0, ACLNN_ERR_PARAM_INVALID, "GroupedMatmulFinalizeRoutingWeightNz dtype must be 0, but is %lld.", (long long)dtype);
    GMM_REQUIRE(x2->rank() >= 2, ACLNN_ERR_PARAM_INVALID, "w's view dimNum should greater than 1, but is %zu.", x2->rank());
    GMM_REQUIRE(!transposeX1 && !transposeX2, ACLNN_ERR_PARAM_INVALID, "GroupedMatmulFinalizeRoutingWeightNz transpose should be false");
    GMM_REQUIRE(x1->format == ACL_FORMAT_ND && x2->format == ACL_FORMAT_FRACTAL_NZ, ACLNN_ERR_PARAM_INVALID,
                "Only support x1: ND, x2: NZ.");
    GMM_REQUIRE(out != nullptr, ACLNN_ERR_PARAM_NULLPTR, "out must not be nullptr.");
    GMM_REQUIRE(offset == nullptr, ACLNN_ERR_PARAM_INVALID, "offset belongs to the int4 weight path, which is not part of this build.");
    // dtypes
    GMM_REQUIRE(x1->dtype == ACL_INT8 && x2->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID,
                "x1 and x2 must be int8 (the int4 weight path is not part of this build).");
    GMM_REQUIRE(scale->dtype == ACL_FLOAT || scale->dtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID,
                "scale dtype must be float32 or bfloat16 (the int64 packed scale is not part of this build).");
    GMM_REQUIRE(rowIndex->dtype == ACL_INT64 || rowIndex->dtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID, "rowIndex dtype must be int64 or int32.");
    GMM_REQUIRE(!bias || bias->dtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID, "bias dtype must be bfloat16.");
    GMM_REQUIRE(!pertokenScale || pertokenScale->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "pertokenScale dtype must be float32.");
    GMM_REQUIRE(groupList->dtype == ACL_INT64, ACLNN_ERR_PARAM_INVALID, "groupList dtype must be int64.");
    GMM_REQUIRE(!sharedInput || sharedInput->dtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID, "sharedInput dtype must be bfloat16.");
    GMM_REQUIRE(!logit || logit->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "logit dtype must be float32.");
    GMM_REQUIRE(out->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "y's dtype should be [DT_FLOAT].");
    // dimension counts (CheckDimRange, :341-377)
    GMM_REQUIRE(x1->rank() == 2, ACLNN_ERR_PARAM_INVALID, "x dim num should be 2, but is %zu.", x1->rank());
    GMM_REQUIRE(x2->rank() == 3 || x2->rank() == 5, ACLNN_ERR_PARAM_INVALID, "w must be viewed as [e, k, n] or as [e, n/32, k/16, 16, 32].");
    GMM_REQUIRE(scale->rank() == 2, ACLNN_ERR_PARAM_INVALID, "scale dim num should be 2.");
    GMM_REQUIRE(!pertokenScale || pertokenScale->rank() == 1, ACLNN_ERR_PARAM_INVALID, "pertokenScale dim num should be 1.");
    GMM_REQUIRE(groupList->rank() == 1, ACLNN_ERR_PARAM_INVALID, "groupList dim num should be 1.");
    GMM_REQUIRE(!sharedInput || sharedInput->rank() == 2, ACLNN_ERR_PARAM_INVALID, "sharedInput dim num should be 2.");
    GMM_REQUIRE(!logit || logit->rank() == 1, ACLNN_ERR_PARAM_INVALID, "logit dim num should be 1.");
    GMM_REQUIRE(rowIndex->rank() == 1, ACLNN_ERR_PARAM_INVALID, "rowIndex dim num should be 1.");
    GMM_REQUIRE(!bias || bias->rank() == 2, ACLNN_ERR_PARAM_INVALID, "bias dim num should be 2.");
    // shapes
    const int64_t M = x1->dim(0), K = x1->dim(1), E = x2->dim(0);
    int64_t wK, N;
    if (x2->rank() == 5) {
        GMM_REQUIRE(x2->dim(3) == 16 && x2->dim(4) == 32, ACLNN_ERR_PARAM_INVALID, "a 5-dimensional w must be [e, n/32, k/16, 16, 32].");
        wK = x2->dim(2) * 16; N = x2->dim(1) * 32;
    } else {
        wK = x2->dim(1); N = x2->dim(2);
        // the storage must hold the fractal form of the view (CheckWeightNzFormat :891-911, CheckShapeForWeightNz :499-518)
        GMM_REQUIRE(x2->storage_dims.size() >= 5, ACLNN_ERR_PARAM_INVALID,
                    "x2's storage shape must be the FRACTAL_NZ form [e, n/32, k/16, 16, 32] of its view.");
        int64_t prod = 1;
        for (int64_t d : x2->storage_dims) prod *= d;
        GMM_REQUIRE(prod == E * ((N + 31) / 32) * ((wK + 15) / 16) * 16 * 32, ACLNN_ERR_PARAM_INVALID,
                    "x2's format only support NZ, but x2's storage shape is not the fractal form of its view.");
        GMM_REQUIRE(x2->storage_dims[x2->storage_dims.size() - 3] * 16 == (K + 15) / 16 * 16, ACLNN_ERR_PARAM_INVALID,
                    "AlignedK1 value is not matched with k1 value times 16.");
    }
    GMM_REQUIRE(K == wK, ACLNN_ERR_PARAM_INVALID, "x1 k dim and x2 k dim should be same, but x1 is %lld, x2 is %lld.", (long long)K, (long long)wK);
    GMM_REQUIRE(K % 16 == 0 && N % 32 == 0 && N >= 256, ACLNN_ERR_PARAM_INVALID,
                "k dim %lld and n dim %lld do not support. only support k mod 16 equal 0, n mod 32 equal 0 and n bigger or equal 256",
                (long long)K, (long long)N);
    GMM_REQUIRE(out->rank() == 2, ACLNN_ERR_PARAM_INVALID, "Out dim num should be equal to 2, but is %zu.", out->rank());
    const int64_t BS = out->dim(0);
    GMM_REQUIRE(BS <= M && BS >= 0, ACLNN_ERR_PARAM_INVALID, "Out 1st dim should be less than or equal to x MDim , but out 1st dim is %lld", (long long)BS);
    GMM_REQUIRE(out->dim(1) == N, ACLNN_ERR_PARAM_INVALID, "Out 2nd dim should be equal to weight NDim.");
    GMM_REQUIRE(sharedInputOffset >= 0, ACLNN_ERR_PARAM_INVALID, "sharedInputOffset should bigger than or equal to 0");
    GMM_REQUIRE(groupListType == 1, ACLNN_ERR_PARAM_INVALID, "groupListType is 1, but is %lld", (long long)groupListType);
    GMM_REQUIRE(scale->dim(0) == E && scale->dim(1) == N, ACLNN_ERR_PARAM_INVALID, "Scale must be [%lld, %lld].", (long long)E, (long long)N);
    GMM_REQUIRE(!bias || (bias->dim(0) == E && bias->dim(1) == N), ACLNN_ERR_PARAM_INVALID, "bias must be [%lld, %lld].", (long long)E, (long long)N);
    GMM_REQUIRE(!pertokenScale || pertokenScale->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "pertokenScale fisrt dim should equal to x MDim %lld.", (long long)M);
    GMM_REQUIRE(groupList->dim(0) == E, ACLNN_ERR_PARAM_INVALID, "groupList fisrt dim should equal to weight EDim %lld.", (long long)E);
    const int64_t sharedRows = sharedInput ? sharedInput->dim(0) : 0;
    GMM_REQUIRE(!sharedInput || (sharedRows <= BS && sharedInput->dim(1) == N), ACLNN_ERR_PARAM_INVALID,
                "shareInput fisrt dim should less than or equal to outputBS %lld, last dim should equal to weight NDim %lld.", (long long)BS, (long long)N);
    GMM_REQUIRE(!logit || logit->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "logit fisrt dim should equal to x MDim %lld.", (long long)M);
    GMM_REQUIRE(rowIndex->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "rowIndex fisrt dim should equal to x MDim %lld.", (long long)M);
    GMM_REQUIRE(sharedInputOffset + sharedRows <= BS, ACLNN_ERR_PARAM_INVALID,
                "shareInputOffset add shareInputDim should be less than or equal to outputBS.");
    GMM_REQUIRE(!x1->empty() && !x2->empty() && !scale->empty() && !groupList->empty() && !rowIndex->empty() &&
                    !(pertokenScale && pertokenScale->empty()) && !(sharedInput && sharedInput->empty()) && !(logit && logit->empty()),
                ACLNN_ERR_PARAM_INVALID, "GroupedMatmulFinalizeRouting WeightNz do not support input tensor size is 0.");
    // formats
    for (const aclTensor *t : {scale, bias, pertokenScale, groupList, sharedInput, logit, rowIndex, (const aclTensor *)out})
        GMM_REQUIRE(!t || t->format == ACL_FORMAT_ND, ACLNN_ERR_PARAM_INVALID, "every tensor but x2 must have format ND.");
    if (tuningConfig && !tuningConfig->values.empty())
        GMM_REQUIRE(tuningConfig->values[0] >= 0 && tuningConfig->values[0] <= M, ACLNN_ERR_PARAM_INVALID,
                    "Invalid tuningConfigOptional (%lld)! It should be a non-negative num and smaller than (%lld)",
                    (long long)tuningConfig->values[0], (long long)M);
    GMM_REQUIRE(E <= kMaxGroupListLen, ACLNN_ERR_PARAM_INVALID, "more than %lld experts.", (long long)kMaxGroupListLen);
    GMM_REQUIRE(K <= kMaxInnerAxis && N <= kMaxInnerAxis, ACLNN_ERR_PARAM_INVALID, "k and n must not exceed %lld.", (long long)kMaxInnerAxis);

    aclOpExecutor *e = new_executor(kOp);
    GMM_REQUIRE(e != nullptr, ACLNN_ERR_INNER_CREATE_EXECUTOR, "cannot create executor.");
    if (out->empty()) return finish_phase1(e, workspaceSize, executor);
    Problem &p = e->problem;
    bind_tensor(e, x1, &p.x, false);
    bind_tensor(e, x2, &p.w, false, true);   // the fractal storage is read as it lies
    bind_tensor(e, scale, &p.w_scale, false);
    p.w_scale_dtype = (int)scale->dtype;
    bind_tensor(e, pertokenScale, &p.x_scale, false);
    bind_tensor(e, bias, &p.bias, false);
    p.bias_dtype = bias ? kBF16 : kNone;
    bind_tensor(e, groupList, &p.group_list, false);
    p.gl_len = (int)E;
    p.gl_type = 1;
    p.M = M; p.K = K; p.N = N; p.E = E;
    p.w_layout = 2;
    p.mode = kModeDequantBf16;
    bind_tensor(e, out, &p.out0, true);
    p.combine = 1;
    bind_tensor(e, logit, &p.logit, false);
    bind_tensor(e, rowIndex, &p.row_index, false);
    p.row_index_i32 = rowIndex->dtype == ACL_INT32;
    p.scatter_add = (sharedInput || logit) ? 1 : 0;   // grouped_matmul_finalize_routing_base_tiling.cpp:296-300
    p.out_rows = BS;
    bind_tensor(e, sharedInput, &p.shared_input, false);
    p.shared_rows = sharedRows;
    p.shared_offset = sharedInputOffset;
    p.shared_weight = sharedInputWeight;
    e->kind = aclOpExecutor::kGmm;
    make_plan(p, &e->plan);
    return finish_phase1(e, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNzGetWorkspaceSize(
    const aclTensor *x1, const aclTensor *x2, const aclTensor *scale, const aclTensor *bias, const aclTensor *pertokenScaleOptional,
    const aclTensor *groupList, const aclTensor *sharedInput, const aclTensor *logit, const aclTensor *rowIndex, int64_t dtype,
    float sharedInputWeight, int64_t sharedInputOffset, bool transposeX1, bool transposeX2, int64_t groupListType, aclTensor *out,
    uint64_t *workspaceSize, aclOpExecutor **executor)
{
    return finalize_routing_phase1("aclnnGroupedMatmulFinalizeRoutingWeightNz", x1, x2, scale, bias, nullptr, pertokenScaleOptional,
                                   groupList, sharedInput, logit, rowIndex, dtype, sharedInputWeight, sharedInputOffset, transposeX1,
                                   transposeX2, groupListType, nullptr, out, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNz(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor,
                                                      aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulFinalizeRoutingWeightNz", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNzV2GetWorkspaceSize(
    const aclTensor *x1, aclTensor *x2, const aclTensor *scale, const aclTensor *bias, const aclTensor *offsetOptional,
    const aclTensor *antiquantScaleOptional, const aclTensor *antiquantOffsetOptional, const aclTensor *pertokenScaleOptional,
    const aclTensor *groupList, const aclTensor *sharedInput, const aclTensor *logit, const aclTensor *rowIndex, int64_t dtype,
    float sharedInputWeight, int64_t sharedInputOffset, bool transposeX1, bool transposeX2, int64_t groupListType,
    const aclIntArray *tuningConfigOptional, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor)
{
    (void)antiquantScaleOptional; (void)antiquantOffsetOptional;  // unused in the reference too (:1007-1008)
    return finalize_routing_phase1("aclnnGroupedMatmulFinalizeRoutingWeightNzV2", x1, x2, scale, bias, offsetOptional,
                                   pertokenScaleOptional, groupList, sharedInput, logit, rowIndex, dtype, sharedInputWeight,
                                   sharedInputOffset, transposeX1, transposeX2, groupListType, tuningConfigOptional, out, workspaceSize,
                                   executor);
}

aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNzV2(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor,
                                                        aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulFinalizeRoutingWeightNzV2", workspace, workspaceSize, executor, stream);
}

// Shared first phase of aclnnGroupedMatmulSwigluQuant and its WeightNZ twin
// (aclnnGroupedMatmulSwigluQuantGetWorkspaceSizeCommon, aclnn_grouped_matmul_swiglu_quant.cpp:411-465).
static aclnnStatus swiglu_phase1(const char *kOp, bool force_nz, const aclTensor *x, const aclTensor *weight, const aclTensor *bias,
                                 const aclTensor *offset, const aclTensor *weightScale, const aclTensor *xScale,
                                 const aclTensor *groupList, aclTensor *output, aclTensor *outputScale, aclTensor *outputOffset,
                                 uint64_t *workspaceSize, aclOpExecutor **executor)
{
    clear_error();
    PhaseRange phase_range(kOp, 1);
    (void)bias; (void)offset; (void)outputOffset;  // accepted and ignored, as in the reference (:86-104)
    // OP_CHECK_COMM_INPUT + CheckNotNull
    GMM_REQUIRE(workspaceSize != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspaceSize must not be nullptr.");
    GMM_REQUIRE(executor != nullptr, ACLNN_ERR_PARAM_NULLPTR, "executor must not be nullptr.");
    GMM_REQUIRE(x != nullptr, ACLNN_ERR_PARAM_NULLPTR, "x must not be nullptr.");
    GMM_REQUIRE(weight != nullptr, ACLNN_ERR_PARAM_NULLPTR, "weight must not be nullptr.");
    GMM_REQUIRE(weightScale != nullptr, ACLNN_ERR_PARAM_NULLPTR, "weightScale must not be nullptr.");
    GMM_REQUIRE(xScale != nullptr, ACLNN_ERR_PARAM_NULLPTR, "xScale must not be nullptr.");
    GMM_REQUIRE(groupList != nullptr, ACLNN_ERR_PARAM_NULLPTR, "groupList must not be nullptr.");
    GMM_REQUIRE(output != nullptr, ACLNN_ERR_PARAM_NULLPTR, "output must not be nullptr.");
    GMM_REQUIRE(outputScale != nullptr, ACLNN_ERR_PARAM_NULLPTR, "outputScale must not be nullptr.");
    // CheckInputOutDims_A8W8
    GMM_REQUIRE(x->rank() == 2, ACLNN_ERR_PARAM_INVALID, "x dim num should be 2, but now is %zu.", x->rank());
    const bool w_nz = force_nz || weight->format == ACL_FORMAT_FRACTAL_NZ;
    GMM_REQUIRE(w_nz || !is_private_format(weight->format), ACLNN_ERR_PARAM_INVALID, "weight format must be ND or FRACTAL_NZ.");
    if (force_nz)
        GMM_REQUIRE(weight->storage_dims.size() == 5, ACLNN_ERR_PARAM_INVALID,
                    "The dimnum of storageShape for second input (weight) must be 5, but is %zu.", weight->storage_dims.size());
    const bool nz_view = w_nz && weight->rank() == 5;
    GMM_REQUIRE(nz_view || weight->rank() == 3, ACLNN_ERR_PARAM_INVALID, "weight dim num should be 3 (ND) or 5 (FRACTAL_NZ), but now is %zu.", weight->rank());
    GMM_REQUIRE(weightScale->rank() == 2, ACLNN_ERR_PARAM_INVALID, "weightScale dim num should be 2, but now is %zu.", weightScale->rank());
    GMM_REQUIRE(xScale->rank() == 1, ACLNN_ERR_PARAM_INVALID, "xScale dim num should be 1, but now is %zu.", xScale->rank());
    GMM_REQUIRE(groupList->rank() == 1, ACLNN_ERR_PARAM_INVALID, "groupList dim num should be 1, but now is %zu.", groupList->rank());
    GMM_REQUIRE(output->rank() == 2, ACLNN_ERR_PARAM_INVALID, "output dim num should be 2, but now is %zu.", output->rank());
    GMM_REQUIRE(outputScale->rank() == 1, ACLNN_ERR_PARAM_INVALID, "outputScale dim num should be 1, but now is %zu.", outputScale->rank());
    // CheckInputOutShape_A8W8
    const int64_t M = x->dim(0), K = x->dim(1), N = weightScale->dim(1), E = weight->dim(0);
    GMM_REQUIRE(N % 2 == 0, ACLNN_ERR_PARAM_INVALID, "aclnnGroupedMatmulSwiGluQuant, N is %lld , not an even number.", (long long)N);
    if (nz_view)
        GMM_REQUIRE(weight->dim(1) == N / 32 && weight->dim(2) == K / 16 && weight->dim(3) == 16 && weight->dim(4) == 32 && N % 32 == 0 && K % 16 == 0,
                    ACLNN_ERR_PARAM_INVALID, "weight shape must be [%lld, %lld, %lld, 16, 32].", (long long)E, (long long)(N / 32), (long long)(K / 16));
    else
        GMM_REQUIRE(weight->dim(1) == K && weight->dim(2) == N, ACLNN_ERR_PARAM_INVALID, "weight shape must be [%lld, %lld, %lld].", (long long)E, (long long)K, (long long)N);
    if (w_nz)
        GMM_REQUIRE(K % 16 == 0 && N % 32 == 0, ACLNN_ERR_PARAM_INVALID, "a FRACTAL_NZ weight needs K %% 16 == 0 and N %% 32 == 0 on this build.");
    GMM_REQUIRE(weightScale->dim(0) == E, ACLNN_ERR_PARAM_INVALID, "weightScale shape must be [%lld, %lld].", (long long)E, (long long)N);
    GMM_REQUIRE(xScale->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "xScale shape must be [%lld].", (long long)M);
    GMM_REQUIRE(output->dim(0) == M && output->dim(1) == N / 2, ACLNN_ERR_PARAM_INVALID, "output shape must be [%lld, %lld].", (long long)M, (long long)(N / 2));
    GMM_REQUIRE(outputScale->dim(0) == M, ACLNN_ERR_PARAM_INVALID, "outputScale shape must be [%lld].", (long long)M);
    const int64_t glLen = groupList->dim(0);
    GMM_REQUIRE(glLen <= E, ACLNN_ERR_PARAM_INVALID,
                "Length of 'groupList' out of range (expected to be in range of [1, %lld], but got %lld)", (long long)E, (long long)glLen);
    GMM_REQUIRE(N <= kSwigluNLimit, ACLNN_ERR_PARAM_INVALID, "N(%lld) is greater than %lld.", (long long)N, (long long)kSwigluNLimit);
    GMM_REQUIRE(K < kSwigluKLimit, ACLNN_ERR_PARAM_INVALID, "The tail axis dimension of input0(x) is %lld, which need lower than %lld.", (long long)K, (long long)kSwigluKLimit);
    // CheckDtypeValid
    GMM_REQUIRE(x->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID, "x dtype must be int8.");
    GMM_REQUIRE(weight->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID, "weight dtype must be int8 (the int4 path is not part of this build).");
    GMM_REQUIRE(weightScale->dtype == ACL_FLOAT || weightScale->dtype == ACL_FLOAT16 || weightScale->dtype == ACL_BF16,
                ACLNN_ERR_PARAM_INVALID, "weightScale dtype must be float32, float16 or bfloat16.");
    GMM_REQUIRE(xScale->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "xScale dtype must be float32.");
    GMM_REQUIRE(groupList->dtype == ACL_INT64, ACLNN_ERR_PARAM_INVALID, "groupList dtype must be int64.");
    GMM_REQUIRE(output->dtype == ACL_INT8, ACLNN_ERR_PARAM_INVALID, "output dtype must be int8.");
    GMM_REQUIRE(outputScale->dtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "outputScale dtype must be float32.");
    GMM_REQUIRE(!is_private_format(x->format) && !is_private_format(output->format), ACLNN_ERR_PARAM_INVALID,
                "x / output Format Not support Private Format.");
    GMM_REQUIRE(glLen <= kMaxGroupListLen, ACLNN_ERR_PARAM_INVALID, "groupList longer than %lld.", (long long)kMaxGroupListLen);
    GMM_REQUIRE(K > 0 || output->empty(), ACLNN_ERR_PARAM_INVALID, "k must be positive (an empty reduction has no row maximum to quantise by).");

    aclOpExecutor *e = new_executor(kOp);
    GMM_REQUIRE(e != nullptr, ACLNN_ERR_INNER_CREATE_EXECUTOR, "cannot create executor.");
    // Empty tensors (aclnn_grouped_matmul_swiglu_quant.cpp:425-429)
    if (output->empty() || groupList->empty() || outputScale->empty()) return finish_phase1(e, workspaceSize, executor);
    Problem &p = e->problem;
    bind_tensor(e, x, &p.x, false);
    bind_tensor(e, weight, &p.w, false, w_nz);
    bind_tensor(e, weightScale, &p.w_scale, false);
    p.w_scale_dtype = (int)weightScale->dtype;
    bind_tensor(e, xScale, &p.x_scale, false);
    bind_tensor(e, groupList, &p.group_list, false);
    p.gl_len = (int)glLen;
    p.gl_type = 0;
    p.M = M; p.K = K; p.N = N; p.E = E;
    p.w_layout = w_nz ? 2 : 0;
    p.mode = kModeSwigluQuant;
    bind_tensor(e, output, &p.out0, true);
    bind_tensor(e, outputScale, &p.out1, true);
    e->kind = aclOpExecutor::kGmm;
    make_plan(p, &e->plan);
    return finish_phase1(e, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulSwigluQuantGetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *bias,
                                                          const aclTensor *offset, const aclTensor *weightScale,
                                                          const aclTensor *xScale, const aclTensor *groupList,
                                                          aclTensor *output, aclTensor *outputScale, aclTensor *outputOffset,
                                                          uint64_t *workspaceSize, aclOpExecutor **executor)
{
    return swiglu_phase1("aclnnGroupedMatmulSwigluQuant", false, x, weight, bias, offset, weightScale, xScale, groupList, output,
                         outputScale, outputOffset, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulSwigluQuant(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor, aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulSwigluQuant", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnGroupedMatmulSwigluQuantWeightNZGetWorkspaceSize(const aclTensor *x, const aclTensor *weight, const aclTensor *bias,
                                                                  const aclTensor *offset, const aclTensor *weightScale,
                                                                  const aclTensor *xScale, const aclTensor *groupList,
                                                                  aclTensor *output, aclTensor *outputScale,
                                                                  aclTensor *outputOffset, uint64_t *workspaceSize,
                                                                  aclOpExecutor **executor)
{
    return swiglu_phase1("aclnnGroupedMatmulSwigluQuantWeightNZ", true, x, weight, bias, offset, weightScale, xScale, groupList,
                         output, outputScale, outputOffset, workspaceSize, executor);
}

aclnnStatus aclnnGroupedMatmulSwigluQuantWeightNZ(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor,
                                                  aclrtStream stream)
{
    return run_executor("aclnnGroupedMatmulSwigluQuantWeightNZ", workspace, workspaceSize, executor, stream);
}

aclnnStatus gmmB200CheckStatus(const void *workspace, uint64_t workspaceSize, aclrtStream stream, int32_t record[4])
{
    clear_error();
    int32_t rec[4] = {0, 0, 0, 0};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t ce;
    if (workspace && workspaceSize >= sizeof(rec)) {
        ce = cudaMemcpyAsync(rec, workspace, sizeof(rec), cudaMemcpyDeviceToHost, s);
        if (ce != cudaSuccess) return fail(ACLNN_ERR_RUNTIME_ERROR, "status copy failed: %s", cudaGetErrorString(ce));
    }
    ce = cudaStreamSynchronize(s);
    if (ce != cudaSuccess) return fail(ACLNN_ERR_RUNTIME_ERROR, "stream failed: %s", cudaGetErrorString(ce));
    if (record) std::memcpy(record, rec, sizeof(rec));
    if (rec[0] != 0)
        return fail(ACLNN_ERR_RUNTIME_ERROR, "kernel reported status %d (CTA %d, role %d, detail %d)", rec[0], rec[1], rec[2], rec[3]);
    return ACLNN_SUCCESS;
}

// ------------------------------------------------------------------------------------------------------------
// Flat entry points
// ------------------------------------------------------------------------------------------------------------

static aclnnStatus flat_sizes_ok(int64_t m, int64_t k, int64_t n, int64_t e)
{
    GMM_REQUIRE(m >= 0 && k > 0 && n > 0 && e > 0, ACLNN_ERR_PARAM_INVALID, "m, k, n, e must be positive (m may be 0).");
    GMM_REQUIRE(m <= 0x7fffffffll / 2, ACLNN_ERR_PARAM_INVALID, "m must not exceed %lld rows.", 0x7fffffffll / 2);
    GMM_REQUIRE(k <= kMaxInnerAxis && n <= kMaxInnerAxis, ACLNN_ERR_PARAM_INVALID, "k and n must not exceed %lld.", (long long)kMaxInnerAxis);
    return ACLNN_SUCCESS;
}

// Workspace for any pointer alignment: the tensor-core layout is a superset of the CUDA-core one.
static uint64_t flat_ws(int64_t m, int64_t k, int64_t n, int64_t e, int mode)
{
    Problem p;
    p.x = reinterpret_cast<const int8_t *>(uintptr_t(256));
    p.w = p.x; p.w_scale = p.x; p.out0 = const_cast<int8_t *>(p.x); p.out1 = p.out0;
    p.M = m; p.K = k; p.N = n; p.E = e; p.gl_len = (int)(e < kMaxGroupListLen ? e : kMaxGroupListLen); p.mode = mode;
    Plan a;
    make_plan(p, &a);
    uint64_t best = a.ws_bytes;
    p.x = reinterpret_cast<const int8_t *>(uintptr_t(1));  // forces the CUDA-core path
    make_plan(p, &a);
    return best > a.ws_bytes ? best : a.ws_bytes;
}

aclnnStatus gmmB200GroupedMatmulW8A8WorkspaceSize(int64_t m, int64_t k, int64_t n, int64_t e, int32_t yDtype, uint64_t *workspaceSize)
{
    clear_error();
    GMM_REQUIRE(workspaceSize != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspaceSize must not be nullptr.");
    aclnnStatus rc = flat_sizes_ok(m, k, n, e);
    if (rc != ACLNN_SUCCESS) return rc;
    GMM_REQUIRE(yDtype == ACL_BF16 || yDtype == ACL_FLOAT16 || yDtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID, "yDtype must be bfloat16, float16 or int32.");
    *workspaceSize = flat_ws(m, k, n, e, yDtype == ACL_INT32 ? kModeInt32 : kModeDequantBf16);
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200GroupedMatmulW8A8(const void *x, const void *weight, const void *scale, int32_t scaleDtype,
                                     const void *perTokenScale, const void *bias, int32_t biasDtype, const void *groupList,
                                     int64_t groupListLen, int32_t groupListType, int64_t m, int64_t k, int64_t n, int64_t e,
                                     int32_t weightTransposed, int32_t actType, const void *outRowIndex, void *const *outPeers,
                                     int32_t numPeers, int64_t outRows, void *y, int32_t yDtype, void *workspace, uint64_t workspaceSize,
                                     aclrtStream stream, const gmmB200LaunchOptions *options)
{
    clear_error();
    PhaseRange phase_range("gmmB200GroupedMatmulW8A8", 2);
    GMM_REQUIRE(x && weight && groupList && (y || numPeers > 0), ACLNN_ERR_PARAM_NULLPTR, "x, weight, groupList and y must not be nullptr.");
    aclnnStatus rc = flat_sizes_ok(m, k, n, e);
    if (rc != ACLNN_SUCCESS) return rc;
    GMM_REQUIRE(yDtype == ACL_BF16 || yDtype == ACL_FLOAT16 || yDtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID, "yDtype must be bfloat16, float16 or int32.");
    GMM_REQUIRE(numPeers >= 0 && numPeers <= 8, ACLNN_ERR_PARAM_INVALID, "numPeers must be in [0, 8].");
    GMM_REQUIRE(outRows >= 0, ACLNN_ERR_PARAM_INVALID, "outRows must not be negative.");
    if (numPeers > 0) {
        GMM_REQUIRE(outPeers && outRowIndex && yDtype == ACL_BF16 && !bias && actType == 0 && perTokenScale, ACLNN_ERR_PARAM_INVALID,
                    "peer output needs outPeers, outRowIndex, a bfloat16 result, a per-token scale, no bias and no activation.");
        for (int i = 0; i < numPeers; ++i)
            GMM_REQUIRE(outPeers[i] && !(reinterpret_cast<uintptr_t>(outPeers[i]) & 15), ACLNN_ERR_PARAM_INVALID, "outPeers[%d] is null or unaligned.", i);
    }
    if (yDtype != ACL_INT32) {
        GMM_REQUIRE(scale != nullptr, ACLNN_ERR_PARAM_NULLPTR, "scale must not be nullptr for a floating-point result.");
        GMM_REQUIRE(scaleDtype == ACL_BF16 || scaleDtype == ACL_FLOAT, ACLNN_ERR_PARAM_INVALID, "scaleDtype must be bfloat16 or float32.");
    }
    GMM_REQUIRE(!bias || biasDtype == ACL_INT32 || biasDtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID, "biasDtype must be int32 or bfloat16.");
    GMM_REQUIRE(groupListType == 0 || groupListType == 1, ACLNN_ERR_PARAM_INVALID, "groupListType should be 0 or 1.");
    GMM_REQUIRE(groupListLen >= 0 && groupListLen <= e && groupListLen <= kMaxGroupListLen, ACLNN_ERR_PARAM_INVALID,
                "groupListLen %lld out of range [0, min(e, %lld)].", (long long)groupListLen, (long long)kMaxGroupListLen);
    GMM_REQUIRE(actType == 0 || actType == 1 || actType == 2 || actType == 4 || actType == 5, ACLNN_ERR_PARAM_INVALID,
                "actType must be 0 (none), 1 (relu), 2 (gelu tanh), 4 (fast gelu) or 5 (silu).");
    GMM_REQUIRE(weightTransposed >= 0 && weightTransposed <= 2, ACLNN_ERR_PARAM_INVALID,
                "weight layout must be 0 ([e,k,n]), 1 ([e,n,k]) or 2 (FRACTAL_NZ).");
    GMM_REQUIRE(weightTransposed != 2 || (k % 16 == 0 && n % 32 == 0), ACLNN_ERR_PARAM_INVALID, "FRACTAL_NZ needs k %% 16 == 0 and n %% 32 == 0.");
    if (m == 0 || groupListLen == 0) return ACLNN_SUCCESS;
    Problem p;
    p.x = static_cast<const int8_t *>(x);
    p.w = static_cast<const int8_t *>(weight);
    p.w_scale = scale; p.w_scale_dtype = scaleDtype;
    p.x_scale = static_cast<const float *>(perTokenScale);
    p.bias = bias; p.bias_dtype = bias ? biasDtype : kNone;
    p.group_list = static_cast<const int64_t *>(groupList);
    p.gl_len = (int)groupListLen; p.gl_type = groupListType;
    p.M = m; p.K = k; p.N = n; p.E = e;
    p.w_layout = weightTransposed;
    p.act_type = yDtype == ACL_INT32 ? 0 : actType;
    p.mode = yDtype == ACL_INT32 ? kModeInt32 : kModeDequantBf16;
    p.out_f16 = yDtype == ACL_FLOAT16 ? 1 : 0;
    p.out0 = y ? y : outPeers[0];
    p.out_row_index = static_cast<const int64_t *>(outRowIndex);
    p.out_rows = outRowIndex ? outRows : 0;
    p.num_peers = numPeers;
    for (int i = 0; i < numPeers; ++i) p.out_peers[i] = outPeers[i];
    rc = convert_options(options, &p.opt);
    if (rc != ACLNN_SUCCESS) return rc;
    Plan plan;
    make_plan(p, &plan);
    GMM_REQUIRE(workspaceSize >= plan.ws_bytes, ACLNN_ERR_PARAM_INVALID, "workspaceSize %llu is smaller than the %llu bytes required.",
                (unsigned long long)workspaceSize, (unsigned long long)plan.ws_bytes);
    GMM_REQUIRE(workspace != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspace must not be nullptr.");
    cudaError_t ce = launch(p, plan, workspace, workspaceSize, static_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return fail(ACLNN_ERR_INNER, "kernel launch failed: %s", cudaGetErrorString(ce));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200GroupedMatmulSwigluQuantWorkspaceSize(int64_t m, int64_t k, int64_t n, int64_t e, uint64_t *workspaceSize)
{
    clear_error();
    GMM_REQUIRE(workspaceSize != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspaceSize must not be nullptr.");
    aclnnStatus rc = flat_sizes_ok(m, k, n, e);
    if (rc != ACLNN_SUCCESS) return rc;
    GMM_REQUIRE(n % 2 == 0 && n <= kSwigluNLimit && k < kSwigluKLimit, ACLNN_ERR_PARAM_INVALID, "n must be even and <= %lld, k < %lld.",
                (long long)kSwigluNLimit, (long long)kSwigluKLimit);
    *workspaceSize = flat_ws(m, k, n, e, kModeSwigluQuant);
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200GroupedMatmulSwigluQuant(const void *x, const void *weight, const void *weightScale, int32_t weightScaleDtype,
                                            const void *xScale, const void *groupList, int64_t groupListLen, int64_t m, int64_t k,
                                            int64_t n, int64_t e, int32_t weightLayout, void *output, void *outputScale,
                                            void *workspace, uint64_t workspaceSize, aclrtStream stream,
                                            const gmmB200LaunchOptions *options)
{
    clear_error();
    PhaseRange phase_range("gmmB200GroupedMatmulSwigluQuant", 2);
    GMM_REQUIRE(x && weight && weightScale && xScale && groupList && output && outputScale, ACLNN_ERR_PARAM_NULLPTR,
                "x, weight, weightScale, xScale, groupList, output and outputScale must not be nullptr.");
    aclnnStatus rc = flat_sizes_ok(m, k, n, e);
    if (rc != ACLNN_SUCCESS) return rc;
    GMM_REQUIRE(n % 2 == 0 && n <= kSwigluNLimit && k < kSwigluKLimit, ACLNN_ERR_PARAM_INVALID, "n must be even and <= %lld, k < %lld.",
                (long long)kSwigluNLimit, (long long)kSwigluKLimit);
    GMM_REQUIRE(weightScaleDtype == ACL_FLOAT || weightScaleDtype == ACL_FLOAT16 || weightScaleDtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID,
                "weightScaleDtype must be float32, float16 or bfloat16.");
    GMM_REQUIRE(groupListLen >= 0 && groupListLen <= e && groupListLen <= kMaxGroupListLen, ACLNN_ERR_PARAM_INVALID,
                "groupListLen %lld out of range [0, min(e, %lld)].", (long long)groupListLen, (long long)kMaxGroupListLen);
    GMM_REQUIRE(weightLayout == 0 || (weightLayout == 2 && k % 16 == 0 && n % 32 == 0), ACLNN_ERR_PARAM_INVALID,
                "weightLayout must be 0 ([e,k,n]) or 2 (FRACTAL_NZ, which needs k %% 16 == 0 and n %% 32 == 0).");
    if (m == 0 || groupListLen == 0) return ACLNN_SUCCESS;
    Problem p;
    p.x = static_cast<const int8_t *>(x);
    p.w = static_cast<const int8_t *>(weight);
    p.w_scale = weightScale; p.w_scale_dtype = weightScaleDtype;
    p.x_scale = static_cast<const float *>(xScale);
    p.group_list = static_cast<const int64_t *>(groupList);
    p.gl_len = (int)groupListLen; p.gl_type = 0;
    p.M = m; p.K = k; p.N = n; p.E = e;
    p.w_layout = weightLayout;
    p.mode = kModeSwigluQuant;
    p.out0 = output; p.out1 = outputScale;
    rc = convert_options(options, &p.opt);
    if (rc != ACLNN_SUCCESS) return rc;
    Plan plan;
    make_plan(p, &plan);
    GMM_REQUIRE(workspaceSize >= plan.ws_bytes, ACLNN_ERR_PARAM_INVALID, "workspaceSize %llu is smaller than the %llu bytes required.",
                (unsigned long long)workspaceSize, (unsigned long long)plan.ws_bytes);
    GMM_REQUIRE(workspace != nullptr, ACLNN_ERR_PARAM_NULLPTR, "workspace must not be nullptr.");
    cudaError_t ce = launch(p, plan, workspace, workspaceSize, static_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return fail(ACLNN_ERR_INNER, "kernel launch failed: %s", cudaGetErrorString(ce));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200GroupedMatmulFinalizeRouting(const void *x, const void *weight, int32_t weightLayout, const void *scale,
                                                int32_t scaleDtype, const void *bias, const void *perTokenScale, const void *groupList,
                                                int64_t groupListLen, int32_t groupListType, const void *sharedInput,
                                                int64_t sharedRows, int64_t sharedOffset, float sharedWeight, const void *logit,
                                                const void *rowIndex, int32_t rowIndexDtype, int64_t m, int64_t k, int64_t n, int64_t e,
                                                void *y, int64_t yRows, void *workspace, uint64_t workspaceSize, aclrtStream stream,
                                                const gmmB200LaunchOptions *options)
{
    clear_error();
    PhaseRange phase_range("gmmB200GroupedMatmulFinalizeRouting", 2);
    GMM_REQUIRE(x && weight && scale && groupList && rowIndex && y, ACLNN_ERR_PARAM_NULLPTR, "x, weight, scale, groupList, rowIndex and y must not be nullptr.");
    GMM_REQUIRE((sharedInput != nullptr) == (logit != nullptr), ACLNN_ERR_PARAM_NULLPTR, "sharedInput and logit come together or not at all.");
    GMM_REQUIRE(m > 0 && m <= 0x7fffffffll / 2 && k > 0 && n > 0 && e > 0 && yRows >= 0 && k <= kMaxInnerAxis && n <= kMaxInnerAxis,
                ACLNN_ERR_PARAM_INVALID, "bad sizes.");
    GMM_REQUIRE(n % 4 == 0, ACLNN_ERR_PARAM_INVALID, "n must be a multiple of 4.");
    GMM_REQUIRE(weightLayout == 0 || (weightLayout == 2 && k % 16 == 0 && n % 32 == 0), ACLNN_ERR_PARAM_INVALID,
                "weightLayout must be 0 ([e,k,n]) or 2 (FRACTAL_NZ, k %% 16 == 0, n %% 32 == 0).");
    GMM_REQUIRE(scaleDtype == ACL_FLOAT || scaleDtype == ACL_BF16, ACLNN_ERR_PARAM_INVALID, "scaleDtype must be float32 or bfloat16.");
    GMM_REQUIRE(rowIndexDtype == ACL_INT64 || rowIndexDtype == ACL_INT32, ACLNN_ERR_PARAM_INVALID, "rowIndexDtype must be int64 or int32.");
    GMM_REQUIRE(groupListType == 0 || groupListType == 1, ACLNN_ERR_PARAM_INVALID, "groupListType must be 0 or 1.");
    GMM_REQUIRE(groupListLen > 0 && groupListLen <= e && groupListLen <= kMaxGroupListLen, ACLNN_ERR_PARAM_INVALID, "bad groupListLen.");
    GMM_REQUIRE(sharedRows >= 0 && sharedOffset >= 0 && sharedOffset + sharedRows <= yRows, ACLNN_ERR_PARAM_INVALID, "shared rows exceed y.");
    Problem p;
    p.x = static_cast<const int8_t *>(x);
    p.w = static_cast<const int8_t *>(weight);
    p.w_scale = scale; p.w_scale_dtype = scaleDtype;
    p.x_scale = static_cast<const float *>(perTokenScale);
    p.bias = bias; p.bias_dtype = bias ? kBF16 : kNone;
    p.group_list = static_cast<const int64_t *>(groupList);
    p.gl_len = (int)groupListLen; p.gl_type = groupListType;
    p.M = m; p.K = k; p.N = n; p.E = e;
    p.w_layout = weightLayout;
    p.mode = kModeDequantBf16;
    p.out0 = y;
    p.combine = 1;
    p.logit = static_cast<const float *>(logit);
    p.row_index = rowIndex;
    p.row_index_i32 = rowIndexDtype == ACL_INT32;
    p.scatter_add = sharedInput ? 1 : 0;
    p.out_rows = yRows;
    p.shared_input = sharedInput; p.shared_rows = sharedRows; p.shared_offset = sharedOffset; p.shared_weight = sharedWeight;
    {
        aclnnStatus orc = convert_options(options, &p.opt);
        if (orc != ACLNN_SUCCESS) return orc;
    }
    Plan plan;
    make_plan(p, &plan);
    GMM_REQUIRE(workspaceSize >= plan.ws_bytes && workspace, ACLNN_ERR_PARAM_INVALID, "workspace of %llu bytes needed.", (unsigned long long)plan.ws_bytes);
    cudaError_t ce = launch(p, plan, workspace, workspaceSize, static_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return fail(ACLNN_ERR_INNER, "gmmB200GroupedMatmulFinalizeRouting: launch failed: %s", cudaGetErrorString(ce));
    return ACLNN_SUCCESS;
}

}  // extern "C"
