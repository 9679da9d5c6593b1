// The whole relation tail of one layer in one launch, for decode batches of a few sequences
// (sm_100a): gathers, product term of the first relation-MLP layer, GELU, second relation-MLP
// layer, per-partner LayerNorm, active-K softmax, weighted sum, residual update, the next
// LayerNorm and (optionally) the next layer's query-side projection.  The relation hidden
// states [pairs, H] never leave the chip and no vendor GEMM is called.
//
//   hidden[b,k,:] = gelu(W_m (o[a_b] * o[p_bk]) + E[a_b, 0:H] + E[p_bk, H:2H])     (16-bit, on chip)
//   raw[b,k,:]    = W_2 hidden[b,k,:] + b_2                                        (fp32, on chip)
//   context[b]    = sum_k w_bk LayerNorm(raw[b,k,:]),  w = softmax over the active partner slots
//   residual[b]  += mix * context[b];  normalized[b] = LayerNorm'(residual[b])
//   query[b]      = W_q normalized[b]                                              (optional)
//
// Geometry.  A thread-block cluster of C = H / 128 CTAs serves up to 64 (sequence, partner)
// pairs; CTA c owns hidden columns [128 c, 128 c + 128).  Its weight slices — W_m[128 c .., :]
// (128 x R) and W_2[:, 128 c ..] (d x 128) — are requested by TMA before the dependency wait and
// stay resident in shared memory.  After the selector's indices arrive every CTA gathers the
// operand rows (multiplied in place into the swizzled B tile) and its 128 columns of the two
// expanded-cache terms, runs the product GEMM with the hidden columns on the TMEM lanes
// (tcgen05.mma, pairs on the TMEM columns), applies GELU and writes its hidden slice as the
// K-major B tile of the second GEMM, whose A operand is the resident W_2 slice: a split-K GEMM
// over the cluster, each CTA holding a partial raw^T [d, pairs] in TMEM.  The partials are dumped
// to shared memory and reduced through distributed shared memory: CTA c pulls the d / C output
// rows it owns from all CTAs in a fixed order (deterministic sums), adds the bias and keeps
// raw[pairs, d / C].  LayerNorm statistics over the full width are combined across the cluster
// from per-CTA (mean, M2) pairs (Chan's parallel variance), which every CTA stores into the
// shared memory of all the others before the barrier (no remote load after it); softmax weights,
// context, residual update and the next LayerNorm follow the same way, and the normalised rows
// are handed to every CTA for its share of the query projection.  Four cluster barriers in total.
//
// Semantics follow src/relation_lm/kernels/relation_reduce.py:72-146 and 360-417 of the
// reference project with the cuBLAS second layer of benchmarks/benchmark_relation_reduce.py:55-64
// in between, and `hidden + sigmoid(mix) * context` of models/stacked_relation.py:124.
// Every wait is bounded; on expiry the kernel sets RLM_DEV_TIMEOUT, still passes every cluster
// barrier (so no CTA waits for a peer that left), frees its TMEM and returns.

#include "relation_layer_tail_body.cuh"

namespace rlm {
namespace {

template <bool kBf16>
__global__ void __launch_bounds__(kLtThreads, 1) relation_layer_tail_kernel(
    const __grid_constant__ CUtensorMap map_wm, const __grid_constant__ CUtensorMap map_w2,
    const LayerTailArgs a) {
    extern __shared__ __align__(1024) unsigned char lt_smem_raw[];
    layer_tail_body<kBf16>(map_wm, map_w2, a, lt_smem_raw, NoStage{});
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_layer_tail_supported(int n_seq, int k_out, int relation_dim, int hidden_dim,
                                                 int d_model, int n_query, int dtype) {
    using namespace rlm;
    LayerTailArgs a{};
    a.n_seq = n_seq; a.k_out = k_out; a.max_t = 1; a.rdim = relation_dim; a.hdim = hidden_dim; a.d = d_model;
    a.n_query = n_query; a.dtype = dtype;
    a.query_weight = n_query > 0 ? &a : nullptr;      // only tested for NULL
    a.query = n_query > 0 ? &a : nullptr;
    if (lt_validate(a) != RLM_OK) return 0;
    const int cluster = hidden_dim / kLtHC;
    auto kernel = dtype == RLM_BF16 ? relation_layer_tail_kernel<true> : relation_layer_tail_kernel<false>;
    if (lt_prepare(reinterpret_cast<const void*>(kernel), cluster) != RLM_OK) return 0;
    // one cluster of this size, with this much shared memory per CTA, must fit the device
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

extern "C" int rlm_relation_layer_tail(
    const void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const float* partner_scores, const void* product_weight,
    const void* second_weight, const void* second_bias, const float* norm_weight, const float* norm_bias,
    const int64_t* position, float norm_eps, float* residual, const float* mix,
    const float* next_norm_weight, const float* next_norm_bias, float next_norm_eps, void* normalized,
    const void* query_weight, void* query, int n_seq, int k_out, int max_t, int relation_dim,
    int hidden_dim, int d_model, int n_query, int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (n_seq == 0) return RLM_OK;
    if (!expanded_cache || !operand_cache || !anchor_index || !partner_index || !partner_scores ||
        !product_weight || !second_weight || !second_bias || !norm_weight || !norm_bias || !position ||
        !residual || !mix || !next_norm_weight || !next_norm_bias || !normalized) {
        set_error("relation_layer_tail: NULL pointer");
        return RLM_ERR_NULL;
    }
    LayerTailArgs a{};
    a.expanded_cache = expanded_cache; a.operand_cache = operand_cache; a.anchor_index = anchor_index;
    a.partner_index = partner_index; a.partner_scores = partner_scores; a.second_bias = second_bias;
    a.norm_w = norm_weight; a.norm_b = norm_bias; a.position = position; a.residual = residual; a.mix = mix;
    a.next_w = next_norm_weight; a.next_b = next_norm_bias; a.normalized = normalized;
    a.query_weight = query_weight; a.query = query; a.status = status; a.eps = norm_eps; a.next_eps = next_norm_eps;
    a.n_seq = n_seq; a.k_out = k_out; a.max_t = max_t; a.rdim = relation_dim; a.hdim = hidden_dim; a.d = d_model;
    a.n_query = query_weight ? n_query : 0; a.dtype = dtype;
    int rc = lt_validate(a);
    if (rc != RLM_OK) return rc;
    if (!aligned16(expanded_cache) || !aligned16(operand_cache) || !aligned16(product_weight) ||
        !aligned16(second_weight) || (query_weight && !aligned16(query_weight))) {
        set_error("relation_layer_tail: caches and weights must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    a.cluster = hidden_dim / kLtHC;
    // a few sequences per cluster: up to four clusters share the work of a small batch (each
    // streams the layer's weights from L2 once), more clusters only for batches beyond 32
    const int most = kLtMaxPairs / k_out < kLtMaxSeq ? kLtMaxPairs / k_out : kLtMaxSeq;
    a.seqs_per_cluster = (n_seq + 3) / 4 < most ? (n_seq + 3) / 4 : most;
    const int clusters = (n_seq + a.seqs_per_cluster - 1) / a.seqs_per_cluster;
    CUtensorMap mwm, mw2;
    if (!make_map(&mwm, product_weight, hidden_dim, relation_dim, relation_dim, kBM, dtype) ||
        !make_map(&mw2, second_weight, d_model, hidden_dim, hidden_dim, kBM, dtype)) {
        set_error("relation_layer_tail: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    auto kernel = dtype == RLM_BF16 ? relation_layer_tail_kernel<true> : relation_layer_tail_kernel<false>;
    rc = lt_prepare(reinterpret_cast<const void*>(kernel), a.cluster);
    if (rc != RLM_OK) return rc;
    const size_t smem_bytes = lt_plan(relation_dim, d_model, kLtMaxPairs).total + 1024;
    launch_kernel_cluster(kernel, dim3(a.cluster, clusters), dim3(kLtThreads),
                          static_cast<unsigned>(a.cluster), smem_bytes, stream, mwm, mw2, a);
    count_launch();
    return check_launch("relation_layer_tail_kernel");
}
