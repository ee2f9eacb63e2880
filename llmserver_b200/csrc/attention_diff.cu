// Differential attention over the paged cache, any sizes, 32-bit arithmetic.
//
// A head attends with two score maps over the same values: its query and its key consist of two units of `dim`
// elements, [map 1 | map 2], and
//     s_m   = (q_m . k_m) * scale,  optionally capped: s_m <- cap * tanh(s_m / cap)
//     a_m   = softmax over the visible keys (s_m) V                                       m = 1, 2
//     o     = a_1 - lambda * a_2
//     out   = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)        (the gate, one number per head, may be absent)
// Query head h reads key/value head h / (Hq / Hkv).  K pages are [page, Hkv, slot, 2 * dim], V pages
// [page, Hkv, slot, value_dim].  The query at position p sees keys max(0, p - window + 1) .. p (window 0: all of them).
//
// One warp per (token, head); keys are visited 32 at a time from the first visible one, each lane owning one key's
// two dot products, so the order of every sum depends only on the query's position: a token's result is the same
// however its prompt was cut into steps and whatever else is in the batch.  This kernel takes every size; it is the
// kernel of the 32-bit path and of bfloat16 shapes the tiled kernel (attention_diff_mma.cu) does not take.
#include "common.cuh"

#define DIFF_MAX_DV 512

template <typename T>
__global__ void attention_diff_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ gate, int gate_stride,
                                      const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                      const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ positions, T* __restrict__ out, int n_q_heads, int n_kv_heads,
                                      int dim, int value_dim, int page_size, int num_pages, float scale, float cap, int window,
                                      float lambda, float eps, float out_scale, int* __restrict__ error_flag) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float q_shared[];  // [warps][2 * dim]
    const int token = blockIdx.x;
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * warps_per_block + warp;
    if (head >= n_q_heads) return;
    const int kv_head = head / (n_q_heads / n_kv_heads);
    const int position = positions[token];
    const int* table = block_tables + (size_t)seq_of_token[token] * max_blocks;
    const int key_dim = 2 * dim;

    float* q_row = q_shared + (size_t)warp * key_dim;
    const T* q_src = q + (size_t)token * q_stride + (size_t)head * key_dim;
    for (int i = lane; i < key_dim; i += 32) q_row[i] = Num<T>::load(q_src + i);
    __syncwarp();

    float acc[2][DIFF_MAX_DV / 32];
#pragma unroll
    for (int i = 0; i < DIFF_MAX_DV / 32; ++i) acc[0][i] = acc[1][i] = 0.0f;
    float running_max[2] = {-INFINITY, -INFINITY}, normaliser[2] = {0.0f, 0.0f};
    const float inverse_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    const int first = (window > 0 && position - window + 1 > 0) ? position - window + 1 : 0;
    for (int base = first; base <= position; base += 32) {
        const int key = base + lane;
        const bool valid = key <= position;
        long long offset = 0;
        float score[2] = {-INFINITY, -INFINITY};
        if (valid) {
            int page = table[key / page_size];
            if ((unsigned)page >= (unsigned)num_pages) {      // no page of the pool: report it, read page 0 instead
                if (error_flag) atomicExch(error_flag, 5);
                page = 0;
            }
            offset = ((long long)page * n_kv_heads + kv_head) * page_size + key % page_size;
            const T* k_row = k_pages + offset * key_dim;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float dot = 0.0f;
                for (int d = 0; d < dim; ++d) dot += q_row[m * dim + d] * Num<T>::load(k_row + m * dim + d);
                dot *= scale;
                score[m] = cap > 0.0f ? cap * tanhf(dot * inverse_cap) : dot;
            }
        }
        float weight[2];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const float new_max = fmaxf(running_max[m], warp_max(score[m]));
            const float correction = expf(running_max[m] - new_max);  // 0 on the first chunk
            weight[m] = valid ? expf(score[m] - new_max) : 0.0f;
            normaliser[m] = normaliser[m] * correction + warp_sum(weight[m]);
#pragma unroll
            for (int i = 0; i < DIFF_MAX_DV / 32; ++i) acc[m][i] *= correction;
            running_max[m] = new_max;
        }
        const int in_chunk = min(32, position - base + 1);
        for (int j = 0; j < in_chunk; ++j) {
            const float w0 = __shfl_sync(0xffffffffu, weight[0], j);
            const float w1 = __shfl_sync(0xffffffffu, weight[1], j);
            const long long row = __shfl_sync(0xffffffffu, offset, j);
            const T* v_row = v_pages + row * value_dim;
#pragma unroll
            for (int i = 0; i < DIFF_MAX_DV / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < value_dim) {
                    const float v = Num<T>::load(v_row + d);
                    acc[0][i] += w0 * v;
                    acc[1][i] += w1 * v;
                }
            }
        }
    }
    const float inverse0 = 1.0f / normaliser[0], inverse1 = lambda / normaliser[1];
    float sum_squares = 0.0f;
#pragma unroll
    for (int i = 0; i < DIFF_MAX_DV / 32; ++i) {
        const int d = lane + 32 * i;
        const float o = d < value_dim ? acc[0][i] * inverse0 - acc[1][i] * inverse1 : 0.0f;
        acc[0][i] = o;
        sum_squares += o * o;
    }
    float factor = rsqrtf(warp_sum(sum_squares) / (float)value_dim + eps) * out_scale;
    if (gate) {
        const float g = Num<T>::load(gate + (size_t)token * gate_stride + head);
        factor *= 1.0f / (1.0f + expf(-g));
    }
    T* dst = out + (size_t)token * n_q_heads * value_dim + (size_t)head * value_dim;
#pragma unroll
    for (int i = 0; i < DIFF_MAX_DV / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) Num<T>::store(dst + d, acc[0][i] * factor);
    }
}

LLM_EXPORT int llm_attention_diff(const void* q, int q_stride, const void* gate, int gate_stride, const void* k_pages,
                                  const void* v_pages, const int* block_tables, int max_blocks, const int* seq_of_token,
                                  const int* positions, void* out, int n_tokens, int n_q_heads, int n_kv_heads, int dim,
                                  int value_dim, int page_size, int num_pages, float scale, float cap, int window, float lambda,
                                  float eps, float out_scale, int* error_flag, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (dim <= 0 || value_dim <= 0 || value_dim > DIFF_MAX_DV) {
        llm_set_error("attention_diff: dim %d must be positive and the value size %d in 1..%d", dim, value_dim, DIFF_MAX_DV);
        return LLM_REFUSED;
    }
    if (num_pages <= 0 || page_size <= 0) {
        llm_set_error("attention_diff: the page pool has %d pages of %d", num_pages, page_size);
        return LLM_REFUSED;
    }
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads) {
        llm_set_error("attention_diff: %d query heads are no multiple of %d kv heads", n_q_heads, n_kv_heads);
        return LLM_REFUSED;
    }
    const int warps = 4;
    dim3 grid(n_tokens, (n_q_heads + warps - 1) / warps);
    const size_t shared = (size_t)warps * 2 * dim * sizeof(float);
    if (shared > 40 * 1024) {
        llm_set_error("attention_diff: units of %d elements need %zu bytes of shared memory", dim, shared);
        return LLM_REFUSED;
    }
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(attention_diff_kernel<T>, grid, warps * 32, shared, stream, (const T*)q, q_stride,
                                  (const T*)gate, gate_stride, (const T*)k_pages, (const T*)v_pages, block_tables, max_blocks,
                                  seq_of_token, positions, (T*)out, n_q_heads, n_kv_heads, dim, value_dim, page_size, num_pages,
                                  scale, cap, window, lambda, eps, out_scale, error_flag)));
    return llm_check_launch("attention_diff");
}
