// Interface between the attention dispatcher and the tcgen05 tensor-core kernel.
#pragma once
#include "come_internal.cuh"

namespace come {

struct AttnArgs {
    const void *q, *k, *v, *bias;
    const int32_t *cu;
    void *out;
    float *lse;
    int dtype;
    int64_t total;            // rows of k / v (all packed tokens)
    int64_t q_begin, q_end;   // global rows that q / out / lse cover: [q_begin, q_end)
    int H, D;
    int64_t q_rs, k_rs, v_rs, o_rs;  // row strides in elements
    int nseg, max_seqlen;
    const int *max_seqlen_dev;  // optional device-resident bound of the longest segment (tightens the work list)
    float scale;
    bool q_free;  // one segment; every query row attends to all of its keys wherever the row lies (cu may be NULL = [0, total])
    // q_free launches may split the key tiles of every work item into k_parts shares (more, shorter items: for launches
    // with few items per SM).  Share p writes out + p * part_o (elements) and lse + p * part_l (floats).
    int k_parts = 1;
    int64_t part_o = 0, part_l = 0;
};

// True when the tensor-core kernel can take the problem (head_dim 64, TMA-compatible addresses and strides).
bool attn_sm100_supported(const AttnArgs &a);
// Caps the CTAs of the following launches of the calling host thread (0 = one CTA per SM).
void attn_sm100_set_cta_limit(int max_ctas);
// Enqueues the tensor-core kernel; returns a COME_* code.
int attn_sm100_launch(const AttnArgs &a, cudaStream_t stream);

}  // namespace come
