// Interface between the attention entry (attn.cu) and the tensor-core prefill path (attn_tc.cu).
#pragma once
#include "runtime.cuh"

namespace detb {

// One prefill attention call after the prep kernel has run in the tile layout: query row (token t, q head h) of kv head
// g = h / rep lives at cell g * Rpad + t * rep + h % rep of qq / sq / mxkey / den / num (Rpad: rows per kv head, a
// multiple of 128; mxkey, den and num cells of real rows are zero).
struct AttnTcCall {
    int M, n_h, n_kv, pos0, capacity, Rpad;
    const int8_t* qq;        // [n_kv][Rpad][256]
    const float* sq;
    unsigned* mxkey;
    long long* den;
    long long* num;          // [n_kv][Rpad][256]
    const int8_t* kq;        // cache
    const float* sk;
    const int16_t* vq;
    const float* qg;
    const float* v_scale;
    float* o;
};
// Whether a call goes through the tensor cores: by shape, mode and workspace size only.
bool attn_tc_applies(int M, int hd, bool rows_mode, bool device_pos, int n_kv, int keys);
void attn_tc_run(const AttnTcCall& c, cudaStream_t q);
void attn_tc_configure(int on, int min_m);

}  // namespace detb
