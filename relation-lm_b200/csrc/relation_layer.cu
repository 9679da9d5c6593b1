// A whole relation layer of a decode step in one launch: the packed selector in front of the
// relation tail, inside the tail's thread-block cluster (see relation_layer_tail_body.cuh and
// relation_select_body.cuh).  A translation unit of its own: see the note in relation_select_body.cuh.

#include "relation_layer_tail_body.cuh"
#include "relation_select_body.cuh"

namespace rlm {
namespace {

// ---- a whole relation layer of a decode step in one launch: the selector in front of the tail
//
// The tail's cluster (relation_layer_tail_body.cuh) has one CTA per 128 hidden columns; the first
// CTAs of the cluster each run the packed selector for one of the cluster's sequences, in the
// shared memory the tail uses from its gathers on (product tile, hidden tile, term rows), while the
// weight slices stream in.  The indices travel through global memory (they are outputs anyway) and
// the cluster barrier.
template <bool kBf16>
struct SelectInFront {
    static constexpr bool kActive = true;
    const SelectArgs* args;
    uint32_t bars;
    __device__ __forceinline__ bool operator()(unsigned char* scratch, uint32_t rank, int s0, int nseq) const {
        if (static_cast<int>(rank) >= nseq) return false;
        // the selector waits for the previous launch itself, as late as its queries allow
        select_row<kBf16, true, false>(*args, s0 + static_cast<int>(rank), scratch, bars);
        return true;
    }
};

template <bool kBf16>
__global__ void __launch_bounds__(kLtThreads, 1) relation_layer_kernel(
    const __grid_constant__ CUtensorMap map_wm, const __grid_constant__ CUtensorMap map_w2,
    const LayerTailArgs tail, const SelectArgs sel) {
    extern __shared__ __align__(1024) unsigned char layer_smem_raw[];
    __shared__ __align__(8) unsigned long long select_bars[4];
    layer_tail_body<kBf16>(map_wm, map_w2, tail, layer_smem_raw, SelectInFront<kBf16>{&sel, smem_u32(select_bars)});
}

int launch_layer(SelectArgs& sel, LayerTailArgs& tail, const void* product_weight, const void* second_weight,
                 void* stream) {
    static_assert(kLtThreads == kThreads, "selector and tail share one CTA shape");
    bool many_rows = false;
    int rc = prepare(sel, many_rows);
    if (rc != RLM_OK) return rc;
    rc = lt_validate(tail);
    if (rc != RLM_OK) return rc;
    if (sel.mode != kPacked || sel.row_batch || sel.row_position || sel.exclude_list || many_rows ||
        sel.n_rows != tail.n_seq || sel.k_out != tail.k_out || sel.max_t != tail.max_t) {
        set_error("relation_layer: the selector must be the decode form over the tail's sequences");
        return RLM_ERR_SHAPE;
    }
    if (sel.query_dtype != tail.dtype || sel.key_dtype != tail.dtype || sel.stats_dtype != tail.dtype) {
        set_error("relation_layer: queries, caches and statistics must share the tail's 16-bit dtype");
        return RLM_ERR_UNSUPPORTED;
    }
    tail.cluster = tail.hdim / kLtHC;
    const int most = kLtMaxPairs / tail.k_out < kLtMaxSeq ? kLtMaxPairs / tail.k_out : kLtMaxSeq;
    tail.seqs_per_cluster = (tail.n_seq + 3) / 4 < most ? (tail.n_seq + 3) / 4 : most;
    if (tail.seqs_per_cluster > tail.cluster) tail.seqs_per_cluster = tail.cluster;   // a selecting CTA per sequence
    const LtPlan whole = lt_plan(tail.rdim, tail.d, kLtMaxPairs);
    if (sel.plan.total > static_cast<int>(whole.total - whole.p)) {
        set_error("relation_layer: the selector's working set does not fit the tail's tile memory (use the two launches)");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(tail.expanded_cache) || !aligned16(tail.operand_cache) || !aligned16(product_weight) ||
        !aligned16(second_weight) || (tail.query_weight && !aligned16(tail.query_weight))) {
        set_error("relation_layer: caches and weights must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    CUtensorMap mwm, mw2;
    if (!make_map(&mwm, product_weight, tail.hdim, tail.rdim, tail.rdim, kBM, tail.dtype) ||
        !make_map(&mw2, second_weight, tail.d, tail.hdim, tail.hdim, kBM, tail.dtype)) {
        set_error("relation_layer: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    auto kernel = tail.dtype == RLM_BF16 ? relation_layer_kernel<true> : relation_layer_kernel<false>;
    rc = lt_prepare(reinterpret_cast<const void*>(kernel), tail.cluster);
    if (rc != RLM_OK) return rc;
    const int clusters = (tail.n_seq + tail.seqs_per_cluster - 1) / tail.seqs_per_cluster;
    const size_t smem_bytes = lt_plan(tail.rdim, tail.d, kLtMaxPairs).total + 1024;
    launch_kernel_cluster(kernel, dim3(tail.cluster, clusters), dim3(kLtThreads), static_cast<unsigned>(tail.cluster),
                          smem_bytes, stream, mwm, mw2, tail, sel);
    count_launch();
    return check_launch("relation_layer_kernel");
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_layer_supported(int n_seq, int k_out, int relation_dim, int hidden_dim, int d_model,
                                           int n_query, int dtype, int max_t, int n_blocks, int buckets,
                                           int local_window, int top_blocks) {
    using namespace rlm;
    LayerTailArgs t{};
    t.n_seq = n_seq; t.k_out = k_out; t.max_t = max_t; t.rdim = relation_dim; t.hdim = hidden_dim; t.d = d_model;
    t.n_query = n_query; t.dtype = dtype;
    t.query_weight = n_query > 0 ? &t : nullptr;      // only tested for NULL
    t.query = n_query > 0 ? &t : nullptr;
    if (lt_validate(t) != RLM_OK) return 0;
    if (n_seq < 1 || max_t < 1 || n_blocks < 1 || buckets < 1 || local_window < 1 || top_blocks < 0 ||
        max_t % n_blocks != 0 || k_out > kMaxKOut)
        return 0;
    const int cluster = hidden_dim / kLtHC;
    const Plan plan = make_plan(n_blocks, max_t / n_blocks, local_window, top_blocks, buckets, dtype_size(dtype),
                                dtype_size(dtype), kPacked, false);
    const LtPlan whole = lt_plan(relation_dim, d_model, kLtMaxPairs);
    if (plan.total > static_cast<int>(whole.total - whole.p)) return 0;
    auto kernel = dtype == RLM_BF16 ? relation_layer_kernel<true> : relation_layer_kernel<false>;
    if (lt_prepare(reinterpret_cast<const void*>(kernel), cluster) != RLM_OK) return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(cluster, 1, 1);
    config.blockDim = dim3(kLtThreads, 1, 1);
    config.dynamicSmemBytes = lt_plan(relation_dim, d_model, kLtMaxPairs).total + 1024;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters > 0 ? 1 : 0;
}

extern "C" int rlm_relation_layer(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    const int64_t* position, int32_t* out_anchor, float* out_anchor_score, int32_t* out_partner,
    float* out_partner_score, int64_t anchor_query_stride, int64_t anchor_router_query_stride,
    int64_t partner_base_stride, int n_blocks, int buckets, int local_window, int top_blocks, int strict_valid,
    int param_dtype,
    const void* expanded_cache, const void* operand_cache, const void* product_weight, const void* second_weight,
    const void* second_bias, const float* norm_weight, const float* norm_bias, float norm_eps, float* residual,
    const float* mix, const float* next_norm_weight, const float* next_norm_bias, float next_norm_eps,
    void* normalized, const void* query_weight, void* query, int n_seq, int k_out, int max_t, int relation_dim,
    int hidden_dim, int d_model, int n_query, int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (n_seq == 0) return RLM_OK;
    if (!expanded_cache || !operand_cache || !product_weight || !second_weight || !second_bias || !norm_weight ||
        !norm_bias || !position || !residual || !mix || !next_norm_weight || !next_norm_bias || !normalized) {
        set_error("relation_layer: NULL pointer");
        return RLM_ERR_NULL;
    }
    SelectArgs a{};
    a.aq_stride = anchor_query_stride; a.arq_stride = anchor_router_query_stride; a.pbase_stride = partner_base_stride;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = anchor_router_query;
    a.anchor_mean = anchor_mean; a.anchor_std = anchor_std; a.anchor_gamma = anchor_gamma; a.anchor_bias = anchor_bias;
    a.partner_base = partner_base; a.partner_anchor_cache = partner_anchor_cache; a.partner_keys = partner_keys;
    a.partner_mean = partner_mean; a.partner_std = partner_std; a.partner_gamma = partner_gamma; a.partner_bias = partner_bias;
    a.position = position; a.out_anchor = out_anchor; a.out_anchor_score = out_anchor_score;
    a.out_partner = out_partner; a.out_partner_score = out_partner_score; a.status = status;
    a.n_rows = n_seq; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out; a.strict_valid = strict_valid != 0;
    a.query_dtype = dtype; a.key_dtype = dtype; a.stats_dtype = dtype; a.param_dtype = param_dtype;
    a.mode = kPacked;
    LayerTailArgs t{};
    t.expanded_cache = expanded_cache; t.operand_cache = operand_cache; t.anchor_index = out_anchor;
    t.partner_index = out_partner; t.partner_scores = out_partner_score; t.second_bias = second_bias;
    t.norm_w = norm_weight; t.norm_b = norm_bias; t.position = position; t.residual = residual; t.mix = mix;
    t.next_w = next_norm_weight; t.next_b = next_norm_bias; t.normalized = normalized;
    t.query_weight = query_weight; t.query = query; t.status = status; t.eps = norm_eps; t.next_eps = next_norm_eps;
    t.n_seq = n_seq; t.k_out = k_out; t.max_t = max_t; t.rdim = relation_dim; t.hdim = hidden_dim; t.d = d_model;
    t.n_query = query_weight ? n_query : 0; t.dtype = dtype;
    return launch_layer(a, t, product_weight, second_weight, stream);
}
