// Input embedding of one decode position (sm_100a): one launch instead of five elementwise ops.
//   x[b, :] = (token_embedding[tokens[b]] + boundary_embedding[boundaries[b]]) * scale
//             + position_embedding[t]
// as src/relation_lm/models/relation_lm.py:130-131 of the reference project does for a whole
// sequence.  The sum of the two embeddings is rounded to the embedding dtype first, as an
// addition of two low-precision tensors is.

#include "rlm_common.cuh"

namespace rlm {
namespace {

struct EmbedArgs {
    const int64_t* tokens;
    const int64_t* boundaries;
    const void* token_table;
    const void* boundary_table;
    const float* position_table;
    const int64_t* position;
    float* out;
    int32_t* status;
    float scale;
    int batch, d_model, vocab, boundary_vocab, max_t, table_dtype;
    // optional LayerNorm outputs of the embedded row (16-bit, [B, d]): two affine parameter sets
    const float* norm_w[2];
    const float* norm_b[2];
    void* norm_out[2];
    float norm_eps;
    int norm_dtype;
};

__global__ void __launch_bounds__(256) decode_embed_kernel(const EmbedArgs a) {
    griddep_sync();
    const int b = blockIdx.x;
    const int64_t tok = a.tokens[b], bnd = a.boundaries[b];
    const int t = static_cast<int>(*a.position);
    if (tok < 0 || tok >= a.vocab || bnd < 0 || bnd >= a.boundary_vocab || t < 0 || t >= a.max_t) {
        if (threadIdx.x == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
        return;
    }
    auto embed = [&](int c) {
        float e = load_scalar(a.token_table, tok * a.d_model + c, a.table_dtype) +
                  load_scalar(a.boundary_table, bnd * a.d_model + c, a.table_dtype);
        if (a.table_dtype == RLM_BF16) e = __bfloat162float(__float2bfloat16_rn(e));
        else if (a.table_dtype == RLM_F16) e = __half2float(__float2half_rn(e));
        return e * a.scale + a.position_table[static_cast<int64_t>(t) * a.d_model + c];
    };
    if (!a.norm_out[0] && !a.norm_out[1]) {
        for (int c = threadIdx.x; c < a.d_model; c += blockDim.x)
            a.out[static_cast<int64_t>(b) * a.d_model + c] = embed(c);
        return;
    }
    // with LayerNorm outputs: four consecutive columns per thread (d_model <= 1024, a multiple of 4)
    __shared__ float scratch[18];
    const int c = 4 * threadIdx.x;
    const bool live = c < a.d_model;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = embed(c + i);
        *reinterpret_cast<float4*>(a.out + static_cast<int64_t>(b) * a.d_model + c) = make_float4(v[0], v[1], v[2], v[3]);
    }
    const size_t row = static_cast<size_t>(b) * a.d_model;
    NormTarget t0{a.norm_w[0], a.norm_b[0], a.norm_out[0] ? static_cast<uint16_t*>(a.norm_out[0]) + row : nullptr};
    NormTarget t1{a.norm_w[1], a.norm_b[1], a.norm_out[1] ? static_cast<uint16_t*>(a.norm_out[1]) + row : nullptr};
    block_layer_norm4(v, live, c, a.d_model, a.norm_eps, t0, t1, a.norm_dtype, scratch);
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_decode_embed(const int64_t* tokens, const int64_t* boundaries,
                                const void* token_table, const void* boundary_table,
                                const float* position_table, const int64_t* position, float scale,
                                float* out, int batch, int d_model, int vocab, int boundary_vocab,
                                int max_t, int table_dtype, const float* norm1_weight,
                                const float* norm1_bias, void* norm1_out, const float* norm2_weight,
                                const float* norm2_bias, void* norm2_out, float norm_eps,
                                int norm_out_dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (batch == 0) return RLM_OK;
    if (!tokens || !boundaries || !token_table || !boundary_table || !position_table || !position || !out) {
        set_error("decode_embed: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (batch < 0 || d_model < 1 || vocab < 1 || boundary_vocab < 1 || max_t < 1) {
        set_error("decode_embed: sizes must be positive");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(table_dtype)) { set_error("decode_embed: unknown dtype code"); return RLM_ERR_DTYPE; }
    if ((norm1_out && (!norm1_weight || !norm1_bias)) || (norm2_out && (!norm2_weight || !norm2_bias))) {
        set_error("decode_embed: a LayerNorm output needs its weight and bias");
        return RLM_ERR_NULL;
    }
    if (norm1_out || norm2_out) {
        if (d_model % 4 != 0 || d_model > 1024 || (norm_out_dtype != RLM_BF16 && norm_out_dtype != RLM_F16)) {
            set_error("decode_embed: LayerNorm outputs need d_model a multiple of 4 up to 1024 and a 16-bit dtype");
            return RLM_ERR_SHAPE;
        }
        if (!aligned16(out) || !aligned16(norm1_weight) || !aligned16(norm1_bias) || !aligned16(norm2_weight) ||
            !aligned16(norm2_bias) || (reinterpret_cast<uintptr_t>(norm1_out) & 7u) ||
            (reinterpret_cast<uintptr_t>(norm2_out) & 7u)) {
            set_error("decode_embed: LayerNorm tensors must be 16-byte aligned");
            return RLM_ERR_ALIGN;
        }
    }
    EmbedArgs a{tokens, boundaries, token_table, boundary_table, position_table, position, out, status,
                scale, batch, d_model, vocab, boundary_vocab, max_t, table_dtype,
                {norm1_weight, norm2_weight}, {norm1_bias, norm2_bias}, {norm1_out, norm2_out}, norm_eps,
                norm_out_dtype};
    launch_kernel(decode_embed_kernel, dim3(batch), dim3(256), 0, stream, a);
    count_launch();
    return check_launch("decode_embed_kernel");
}
