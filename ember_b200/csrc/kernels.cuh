// Internal interface between the C-ABI dispatcher and the kernel families.
#pragma once

#include "common.cuh"

namespace ember {

struct AttnArgs {
    const void *q = nullptr, *k = nullptr, *v = nullptr;
    void *out = nullptr;
    float *lse = nullptr;
    const void *dout = nullptr;
    void *dq = nullptr, *dk = nullptr, *dv = nullptr;
    int bh = 0, lq = 0, lk = 0, d = 0;
    float scale = 1.f;
    int causal = 0;
    int dtype = EMBER_F32;
};

// CUDA-core kernels (attn_simt.cu): float32 math, f32 or bf16 storage, d <= 128.
int simt_attention_fwd(const AttnArgs &a, cudaStream_t s);
int simt_attention_bwd(const AttnArgs &a, float *delta, cudaStream_t s);
int launch_delta(const AttnArgs &a, float *delta, cudaStream_t s);

// tcgen05 kernels (attn_fwd_sm100.cu / attn_bwd_sm100.cu): bf16 storage, d in {64, 128}.
bool sm100_fwd_supported(const AttnArgs &a);
int sm100_attention_fwd(const AttnArgs &a, DeviceState *st, cudaStream_t s);
bool sm100_bwd_supported(const AttnArgs &a);
int sm100_attention_bwd(const AttnArgs &a, float *delta, DeviceState *st, cudaStream_t s);

// Split-KV decode (attn_decode.cu): lq == 1, bf16 or f32 storage, d <= 256 and d % 8 == 0.
int decode_pick_splits(int bh, int lk, int d, int dtype, int sm_count);
size_t decode_workspace_bytes(int bh, int d, int splits);
int decode_attention(const AttnArgs &a, int splits, void *workspace, DeviceState *st, cudaStream_t s);

}  // namespace ember
