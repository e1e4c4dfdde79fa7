// Per-step attention metadata handed from the model runner to the attention layer (mirrors
// include/utils/context.h:7-28 of the reference).  One instance per host thread: each tensor-parallel
// rank runs on its own thread and sets its own context (src/utils/context.cpp:6).
#pragma once

#include "utils/tensor.h"

namespace nano_vllm {

struct Context {
    bool is_prefill = false;
    Tensor cu_seqlens_q;   // [num_seqs + 1] int32, prefill
    Tensor cu_seqlens_k;   // [num_seqs + 1] int32, prefill
    int max_seqlen_q = 0;
    int max_seqlen_k = 0;
    Tensor slot_mapping;   // [tokens] int32, -1 = padding
    Tensor context_lens;   // [batch] int32, decode (includes the token being generated)
    Tensor block_tables;   // [batch, max_blocks] int32, zero padded
};

Context& get_context();
void set_context(const Context& context);
void set_context(bool is_prefill,
                 const Tensor& cu_seqlens_q = Tensor(),
                 const Tensor& cu_seqlens_k = Tensor(),
                 int max_seqlen_q = 0,
                 int max_seqlen_k = 0,
                 const Tensor& slot_mapping = Tensor(),
                 const Tensor& context_lens = Tensor(),
                 const Tensor& block_tables = Tensor());
void reset_context();

}  // namespace nano_vllm
