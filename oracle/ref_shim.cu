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
