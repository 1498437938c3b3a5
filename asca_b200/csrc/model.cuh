// The model object behind asca_model_*: offsets of the tensors in the flat parameter buffer (reference parameter
// order, rust/src/model.rs:593-609), the flat device buffers and the data-parallel state. Shared by model.cu (the
// dataflow) and dp.cu (the gradient exchange).
#pragma once
#include "common.cuh"

#include <vector>

struct Lyr {
    int64_t w_qkv, b_qkv, w_gate, b_gate, w_o, b_o, w1, b1, w2, b2;
};

struct asca_dp;   // dp.cu

struct asca_model {
    int64_t vocab, d, H, L, E, F, n_params;
    int64_t embed, head;
    std::vector<Lyr> lay;
    // offsets of the same tensors in the bf16 copy, each rounded up to 8 elements (16 bytes: TMA base alignment)
    std::vector<Lyr> lay16;
    int64_t embed16 = 0, head16 = 0, n16 = 0;
    std::vector<int64_t> seg16;
    std::vector<int64_t> seg_off;   // tensor offsets in parameter order, + total
    float *params = nullptr, *grads = nullptr, *m = nullptr, *v = nullptr;
    uint32_t adam_counter = 0;
    int compute = ASCA_F32;              // ASCA_BF16: tensor-core products on a bf16 copy of the weights
    __nv_bfloat16* params16 = nullptr;   // refreshed from the f32 master copy whenever that changed
    bool params16_stale = true;
    // decode only: per block the qkv and gate projections side by side, [d x ldq] bf16 + bias [ldq] f32,
    // so that one product feeds the state update
    __nv_bfloat16* dec_w = nullptr;
    float* dec_b = nullptr;
    bool dec_stale = true, dec_pk_stale = true;
    __nv_bfloat16* dec_pk = nullptr;   // decode: every product's weights in the few-row kernel's streaming order
    // asca_model_zero_grads only records the request: the next backward overwrites every gradient tensor instead
    // of adding to it (each tensor is written exactly once per backward), which saves the clearing pass and the
    // read half of the accumulation. Anything that exposes the buffer earlier clears it for real first.
    bool grads_zero_pending = false;
    float grad_scale = 1.0f;   // multiplies dLoss/dlogits: 1 / micro-batches when gradients are accumulated
    // called during the backward, on the host, each time a contiguous range of the gradient buffer has had all its
    // kernels enqueued (one block's tensors, last block first, then embedding + head): the data-parallel
    // exchange of that range can be queued behind them while the rest of the backward is still running
    asca_grad_ready_fn grad_hook = nullptr;
    void* grad_hook_user = nullptr;
    // bf16 mode: let the qkv projection's epilogue normalise q, k and write q, k, v as bf16 where the product runs on
    // CTA pairs (asca_model_set_fused_qkv)
    bool fused_qkv = true;
    // bf16 mode, vocabulary 256: let the head product's epilogue take the cross-entropy (loss and bf16 dlogits) where
    // it runs on CTA pairs and the caller does not ask for the logits (asca_model_set_fused_head)
    bool fused_head = true;
    // data parallelism (dp.cu): the communicator attached to this model and what is in flight on its side stream
    asca_dp* dp = nullptr;
    // set by a sharded optimizer step: the f32 master weights and moments of the other ranks' chunks are not
    // current on this rank until asca_model_dp_gather_master has run; reading them out is refused meanwhile
    bool master_stale = false;
};

// dp.cu -- called from the model's dataflow
// Every kernel writing grads[off, off + cnt) has been enqueued: queue the exchange of the range (no-op unless a
// communicator is attached, armed and has more than one rank).
int asca_dp_grad_ready(asca_ctx* ctx, asca_model* m, int64_t off, int64_t cnt);
// The forward is about to read block `layer`'s bf16 expert weights: wait for their all-gather if one is pending.
int asca_dp_before_expert_weights(asca_ctx* ctx, asca_model* m, int64_t layer);
// Anything else about to read the bf16 weight copy: wait for every pending all-gather.
int asca_dp_wait_all(asca_ctx* ctx, asca_model* m);
void asca_dp_free(asca_model* m);
