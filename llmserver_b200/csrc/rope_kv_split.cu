// Rotary position encoding + paged K/V write for heads whose keys and values differ in size, with a
// magnitude on the rotation.
//
// The packed projection of a token is [Hq * D | Hkv * D | Hkv * Dv]: query and key heads of D elements, value
// heads of Dv.  One warp per (token, head):
//   * Q heads: the first `rotary_dim` elements rotated where they lie (attention reads them there);
//   * K heads: the same, written into the token's slot of the K pages [page, Hkv, slot, D];
//   * V heads: copied into the V pages [page, Hkv, slot, Dv].
// Element i < rotary_dim / 2 pairs with element i + rotary_dim / 2 (or, interleaved, 2i with 2i + 1):
//     (u, v) -> (u c - v s, v c + u s),  c = magnitude * cos(position * inv_freq[i]),  s = magnitude * sin(...)
// so an encoding that stretches its frequencies (and scales cos and sin to make up for it) needs nothing but its
// own inv_freq and magnitude.  Angles, cos, sin and the products are 32-bit; each value is rounded once.
// There is no per-head norm here; `llm_qk_norm_rope_kv_write` is the kernel for equal sizes with one.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_split_kernel(T* __restrict__ qkv, const float* __restrict__ inv_freq, float magnitude,
                                           const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                           const int* __restrict__ block_tables, int max_blocks,
                                           T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q_heads,
                                           int n_kv_heads, int key_dim, int value_dim, int page_size, int num_pages,
                                           int write_cache, int* __restrict__ error_flag, int rotary_dim,
                                           int interleaved, int heads_per_block) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float2 rotation[];   // (c, s) per rotating pair
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warps_per_block = blockDim.x >> 5;
    const int half = rotary_dim >> 1;
    const int position = positions[token];
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float angle = (float)position * inv_freq[i];
            rotation[i] = make_float2(magnitude * cosf(angle), magnitude * sinf(angle));
        }
    }
    __syncthreads();
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    const size_t row_width = (size_t)(n_q_heads + n_kv_heads) * key_dim + (size_t)n_kv_heads * value_dim;
    T* row = qkv + (size_t)token * row_width;
    const int first_head = blockIdx.y * heads_per_block;
    const int end_head = min(first_head + heads_per_block, total_heads);
    for (int head = first_head + (threadIdx.x >> 5); head < end_head; head += warps_per_block) {
        const bool is_q = head < n_q_heads;
        const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
        const int kv_head = is_q ? 0 : (is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads);
        T* src = is_q || is_k ? row + (size_t)head * key_dim
                              : row + (size_t)(n_q_heads + n_kv_heads) * key_dim + (size_t)kv_head * value_dim;
        T* dst = src;
        if (!is_q) {
            if (!write_cache) continue;
            const int page = block_tables[(size_t)seq_of_token[token] * max_blocks + position / page_size];
            if (page < 0 || page >= num_pages) {
                if (lane == 0) atomicExch(error_flag, 1 + token);   // the host turns this into an exception
                continue;
            }
            const size_t slot = ((size_t)page * n_kv_heads + kv_head) * page_size + position % page_size;
            dst = is_k ? k_pages + slot * key_dim : v_pages + slot * value_dim;
        }
        if (!is_q && !is_k) {
            for (int i = lane; i < value_dim; i += 32) dst[i] = src[i];
            continue;
        }
        if (inv_freq) {
            for (int i = lane; i < half; i += 32) {
                const int first = interleaved ? 2 * i : i, second = interleaved ? 2 * i + 1 : half + i;
                const float u = Num<T>::load(src + first), v = Num<T>::load(src + second);
                const float2 r = rotation[i];
                Num<T>::store(dst + first, u * r.x - v * r.y);
                Num<T>::store(dst + second, v * r.x + u * r.y);
            }
        }
        if (dst != src) {      // keys: what does not rotate is copied as it is
            for (int i = (inv_freq ? rotary_dim : 0) + lane; i < key_dim; i += 32) dst[i] = src[i];
        }
    }
}

LLM_EXPORT int llm_rope_kv_write_split(void* qkv, const float* inv_freq, float magnitude, const int* positions,
                                       const int* seq_of_token, const int* block_tables, int max_blocks, void* k_pages,
                                       void* v_pages, int n_tokens, int n_q_heads, int n_kv_heads, int key_dim,
                                       int value_dim, int page_size, int num_pages, int write_cache, int* error_flag,
                                       int rotary_dim, int interleaved, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (inv_freq == nullptr) rotary_dim = 0;
    if (rotary_dim < 0 || rotary_dim > key_dim || rotary_dim % 2) {
        llm_set_error("rope_kv_write_split: rotary_dim must be even and at most the key size %d, got %d", key_dim, rotary_dim);
        return LLM_REFUSED;
    }
    if (key_dim <= 0 || value_dim <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || page_size <= 0 || num_pages <= 0) {
        llm_set_error("rope_kv_write_split: sizes must be positive");
        return LLM_REFUSED;
    }
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    const int warps = n_tokens >= 256 ? 8 : 4;
    const int heads_per_block = n_tokens >= 256 ? total_heads : warps;
    dim3 grid(n_tokens, (total_heads + heads_per_block - 1) / heads_per_block);
    const size_t shared = (size_t)(rotary_dim / 2 + 1) * sizeof(float2);
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(rope_kv_write_split_kernel<T>, grid, warps * 32, shared, stream, (T*)qkv, inv_freq,
                                  magnitude, positions, seq_of_token, block_tables, max_blocks, (T*)k_pages, (T*)v_pages,
                                  n_q_heads, n_kv_heads, key_dim, value_dim, page_size, num_pages, write_cache,
                                  error_flag, rotary_dim, interleaved, heads_per_block)));
    return llm_check_launch("rope_kv_write_split");
}
