// Compiles the reference's own CPU RoPE (example_llmc_rope.cu:19-86) in place,
// without copying it: the reference translation unit is included from where it
// lies and two C entry points are exported around its functions.
// TEST INFRASTRUCTURE ONLY - the result (oracle/_ref/libref_rope.so) validates
// the C restatement in rope_oracle.c and produces the golden vectors.
#define main reference_main
#include "example_llmc_rope.cu"
#undef main

#define REF_EXPORT extern "C" __attribute__((visibility("default")))

REF_EXPORT void ref_precompute_freqs_cis(float* table, int dim, int end, float theta, int use_scaled) {
    precompute_freqs_cis(table, dim, end, theta, use_scaled);
}

REF_EXPORT void ref_apply_rotary_emb_forward(float* out, const float* inp, const float* table,
                                             int B, int T, int n_head, int head_dim) {
    apply_rotary_emb_forward(out, inp, table, B, T, n_head, head_dim);
}

REF_EXPORT void ref_apply_rotary_emb_backward(float* dinp, const float* dout, const float* inp, const float* table,
                                              int B, int T, int n_head, int head_dim) {
    apply_rotary_emb_backward(dinp, dout, inp, table, B, T, n_head, head_dim);
}

// llm.c's naive in-place RoPE kernel (example_llmc_rope.cu:89-121), launched as the reference's launcher does
// (:124-130) but with the query / key-value head counts passed through, on a caller-given stream.  Used only as
// the "naive GPU kernel" line of the benchmark's comparison table.
REF_EXPORT int ref_rope_forward_inplace_kernel1(float* inout, const float* table, int B, int T, int n_q, int n_kv,
                                                int head_dim, int block_size, void* stream) {
    int total_threads = B * T * (n_q + 2 * n_kv) * head_dim / 2;
    int num_blocks = (total_threads + block_size - 1) / block_size;
    rope_forward_inplace_kernel1<<<num_blocks, block_size, 0, (cudaStream_t)stream>>>(inout, table, B, T, n_q, n_kv, head_dim);
    return (int)cudaGetLastError();
}
