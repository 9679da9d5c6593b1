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
    for (int c = threadIdx.x; c < a.d_model; c += blockDim.x) {
        float e = load_scalar(a.token_table, tok * a.d_model + c, a.table_dtype) +
                  load_scalar(a.boundary_table, bnd * a.d_model + c, a.table_dtype);
        if (a.table_dtype == RLM_BF16) e = __bfloat162float(__float2bfloat16_rn(e));
        else if (a.table_dtype == RLM_F16) e = __half2float(__float2half_rn(e));
        a.out[static_cast<int64_t>(b) * a.d_model + c] =
            e * a.scale + a.position_table[static_cast<int64_t>(t) * a.d_model + c];
    }
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_decode_embed(const int64_t* tokens, const int64_t* boundaries,
                                const void* token_table, const void* boundary_table,
                                const float* position_table, const int64_t* position, float scale,
                                float* out, int batch, int d_model, int vocab, int boundary_vocab,
                                int max_t, int table_dtype, int32_t* status, void* stream) {
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
    EmbedArgs a{tokens, boundaries, token_table, boundary_table, position_table, position, out, status,
                scale, batch, d_model, vocab, boundary_vocab, max_t, table_dtype};
    launch_kernel(decode_embed_kernel, dim3(batch), dim3(256), 0, stream, a);
    count_launch();
    return check_launch("decode_embed_kernel");
}
