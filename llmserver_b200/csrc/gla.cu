// Gated linear attention: the recurrence over a step's tokens, with its state in 32-bit per request.
//
// Per head, with key channels i < dim and value channels j < vdim:
//     alpha_t[i] = sigmoid(z_t[i] + b[i]) ^ (1 / tau)         = exp(-softplus(-(z + b)) / tau), formed in 32-bit
//     S_t[i][j]  = alpha_t[i] * S_(t-1)[i][j] + k_t[i] * v_t[j]
//     o_t[j]     = sum_i S_t[i][j] * q_t[i] * q_scale
//     out_t[j]   = o_t[j] / sqrt(mean_j(o_t^2) + eps) * weight[j] * silu(g_t[j])
// q, k, v and g are column ranges of one packed projection row; z is a projection of its own, kept in 32-bit (the
// decay is the one quantity here whose error compounds from token to token).  The state of a
// sequence lives in its slot of `state` [slots, heads, dim, vdim] (float32): it is read when the block starts on the
// sequence's tokens of this step and written back behind the last of them, so a prompt may arrive in portions of any
// size and single decoded tokens continue it.  A slot that a new request takes over is zeroed by the cache manager.
//
// One block per (sequence, head).  A thread owns `R` rows of one column of S in registers; `P` such row partitions
// cover dim.  Tokens are taken sixteen at a time: (1) the block stages their q, k, alpha and v in shared memory, the decay
// and everything else that enters the recurrence in 32-bit; (2) every thread walks the sixteen tokens on its registers
// and leaves its partial o; (3) the warps add the partitions' parts in a fixed order, normalise, gate and store.  The
// order of every sum depends on the sizes alone, so a token's result does not depend on how the prompt was cut or on
// what else is in the batch.
//
// Long portions can also be walked segment by segment in parallel (`llm_gla_recurrent` with a segment length): pass A
// runs every segment but the last from a zero state and leaves its end state and the product of its decays; a scan adds
// them up, S_in(k+1) = D_k S_in(k) + S_local(k), which gives every segment the state it starts from; pass C runs the
// segments again from those states and writes the outputs.  Twice the arithmetic, all of it still 32-bit, on as many
// blocks as there are segments; sums are then grouped by segment, so results agree with the one-pass form to rounding,
// not bit for bit (the 32-bit path keeps the one-pass form).
#include "common.cuh"

#define GLA_TOKENS 16

struct GlaArgs {
    const void* proj;       // [N, row_width]
    int row_width, q_offset, k_offset, v_offset, g_offset;
    const float* z;         // [N, heads * dim], 32-bit in either path
    const float* z_bias;    // [heads * dim] or null
    const void* weight;     // [vdim] norm weight
    float* state;           // [slots, heads, dim, vdim]
    const int* state_slots; // [S]
    const int* q_start;     // [S + 1]
    void* out;              // [N, heads * vdim]
    int heads, dim, vdim, partitions, padded_dim, column_threads;
    float inverse_tau, q_scale, eps;
    int segment, max_segments;   // segmented form: tokens per segment, segments the scratch has room for per sequence
    float* segment_state;        // [S, max_segments, heads, dim, vdim]
    float* segment_decay;        // [S, max_segments, heads, dim]
};

// MODE 0: a sequence's tokens in one pass, from and into its state slot.  1: pass A of the segmented form.  3: pass C.
enum : int { GLA_ONE_PASS = 0, GLA_LOCAL = 1, GLA_OUTPUT = 3 };

// R = 128 comes with 256 threads, where a thread's 128 rows of state fit its registers, and, for sizes nothing else
// takes, with 512 (R given as 129), where they spill: slow, but every size up to 256 x 256 then runs.
template <typename T, typename W, int RR, int MODE>
__global__ void __launch_bounds__(RR == 128 ? 256 : 512, RR <= 16 ? 2 : 1) gla_recurrent_kernel(GlaArgs a) {
    constexpr int R = RR == 129 ? 128 : RR;
    pdl_trigger();
    pdl_wait();
    extern __shared__ float4 gla_shared_raw[];
    float* shared = reinterpret_cast<float*>(gla_shared_raw);
    const int seq = blockIdx.x, head = blockIdx.y;
    int begin = a.q_start[seq], end = a.q_start[seq + 1];
    if (begin >= end) return;
    bool last_segment = true;
    size_t segment_index = 0;
    if (MODE != GLA_ONE_PASS) {
        const int segments = (end - begin + a.segment - 1) / a.segment;
        const int segment = blockIdx.z;
        if (segment >= segments) return;
        last_segment = segment == segments - 1;
        if (MODE == GLA_LOCAL && last_segment) return;      // nobody needs the state a zero start leaves behind the last one
        begin += segment * a.segment;
        end = min(end, begin + a.segment);
        segment_index = ((size_t)seq * a.max_segments + segment) * a.heads + head;
    }
    const int dim = a.dim, vdim = a.vdim, padded = a.padded_dim;
    float* q_s = shared;                                   // [GLA_TOKENS][padded]
    float* k_s = q_s + GLA_TOKENS * padded;
    float* alpha_s = k_s + GLA_TOKENS * padded;
    float* v_s = alpha_s + GLA_TOKENS * padded;            // [GLA_TOKENS][vdim]
    float* part_s = v_s + GLA_TOKENS * vdim;               // [partitions][GLA_TOKENS][vdim]
    const int column = threadIdx.x % a.column_threads, partition = threadIdx.x / a.column_threads;
    const int row0 = partition * R;
    const bool owner = column < vdim && partition < a.partitions;
    const T* proj = (const T*)a.proj;
    const float* z = a.z;

    float S[R];
    float decay[MODE == GLA_LOCAL ? R : 1];      // pass A: the product of the segment's decays, row by row
    float* state = a.state + ((size_t)a.state_slots[seq] * a.heads + head) * dim * vdim;
    float* segment_state = a.segment_state + segment_index * dim * vdim;
    const float* source = MODE == GLA_OUTPUT ? segment_state : state;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        S[i] = (MODE != GLA_LOCAL && owner && row0 + i < dim) ? source[(size_t)(row0 + i) * vdim + column] : 0.0f;
        if (MODE == GLA_LOCAL) decay[i] = 1.0f;
    }

    for (int first = begin; first < end; first += GLA_TOKENS) {
        const int count = min(GLA_TOKENS, end - first);
        __syncthreads();      // the parts of the tokens before have been read
        for (int e = threadIdx.x; e < count * padded; e += blockDim.x) {
            const int t = e / padded, i = e % padded;
            float qv = 0.0f, kv = 0.0f, alpha = 0.0f;
            if (i < dim) {
                const T* row = proj + (size_t)(first + t) * a.row_width;
                qv = Num<T>::load(row + a.q_offset + head * dim + i) * a.q_scale;
                kv = Num<T>::load(row + a.k_offset + head * dim + i);
                float zz = z[(size_t)(first + t) * a.heads * dim + head * dim + i];
                if (a.z_bias) zz += a.z_bias[head * dim + i];
                // log sigmoid(zz) = -softplus(-zz), stable on both sides
                const float log_sigmoid = zz >= 0.0f ? -log1pf(expf(-zz)) : zz - log1pf(expf(zz));
                alpha = expf(log_sigmoid * a.inverse_tau);
            }
            q_s[e] = qv;
            k_s[e] = kv;
            alpha_s[e] = alpha;
        }
        for (int e = threadIdx.x; e < count * vdim; e += blockDim.x) {
            const int t = e / vdim, j = e % vdim;
            v_s[e] = Num<T>::load(proj + (size_t)(first + t) * a.row_width + a.v_offset + head * vdim + j);
        }
        __syncthreads();
        if (owner) {
            for (int t = 0; t < count; ++t) {
                const float vj = v_s[t * vdim + column];
                const float4* q4 = reinterpret_cast<const float4*>(q_s + t * padded + row0);
                const float4* k4 = reinterpret_cast<const float4*>(k_s + t * padded + row0);
                const float4* a4 = reinterpret_cast<const float4*>(alpha_s + t * padded + row0);
                float o = 0.0f;
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 qq = q4[i], kk = k4[i], aa = a4[i];
                    S[4 * i + 0] = fmaf(aa.x, S[4 * i + 0], kk.x * vj);
                    S[4 * i + 1] = fmaf(aa.y, S[4 * i + 1], kk.y * vj);
                    S[4 * i + 2] = fmaf(aa.z, S[4 * i + 2], kk.z * vj);
                    S[4 * i + 3] = fmaf(aa.w, S[4 * i + 3], kk.w * vj);
                    if (MODE == GLA_LOCAL) {
                        decay[4 * i + 0] *= aa.x;
                        decay[4 * i + 1] *= aa.y;
                        decay[4 * i + 2] *= aa.z;
                        decay[4 * i + 3] *= aa.w;
                    } else {
                        o = fmaf(S[4 * i + 0], qq.x, o);
                        o = fmaf(S[4 * i + 1], qq.y, o);
                        o = fmaf(S[4 * i + 2], qq.z, o);
                        o = fmaf(S[4 * i + 3], qq.w, o);
                    }
                }
                if (MODE != GLA_LOCAL) part_s[((size_t)partition * GLA_TOKENS + t) * vdim + column] = o;
            }
        }
        if (MODE == GLA_LOCAL) continue;
        __syncthreads();
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int t = warp; t < count; t += warps) {
            float sum_squares = 0.0f;
            for (int j = lane; j < vdim; j += 32) {
                float o = 0.0f;
                for (int p = 0; p < a.partitions; ++p) o += part_s[((size_t)p * GLA_TOKENS + t) * vdim + j];
                part_s[(size_t)t * vdim + j] = o;      // partition 0's place: each element is read and written by one lane
                sum_squares += o * o;
            }
            const float inverse = rsqrtf(warp_sum(sum_squares) / (float)vdim + a.eps);
            const T* g_row = proj + (size_t)(first + t) * a.row_width + a.g_offset + head * vdim;
            T* dst = (T*)a.out + (size_t)(first + t) * a.heads * vdim + head * vdim;
            for (int j = lane; j < vdim; j += 32) {
                const float g = Num<T>::load(g_row + j);
                const float gate = g / (1.0f + expf(-g));
                Num<T>::store(dst + j, part_s[(size_t)t * vdim + j] * inverse * Num<W>::load((const W*)a.weight + j) * gate);
            }
        }
    }
    if (owner && (MODE == GLA_LOCAL || last_segment)) {
        float* target = MODE == GLA_LOCAL ? segment_state : state;
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (row0 + i < dim) target[(size_t)(row0 + i) * vdim + column] = S[i];
        if (MODE == GLA_LOCAL && column == 0) {
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (row0 + i < dim) a.segment_decay[segment_index * dim + row0 + i] = decay[i];
        }
    }
}

// The scan between the passes: per (sequence, head), S_in(0) is the slot's state and S_in(k + 1) = D_k S_in(k) + S_local(k);
// S_in(k) takes S_local(k)'s place in the scratch.  One thread per cell of S: the cells are independent, and the
// segments' values are loaded a few ahead of the chain of multiply-adds that needs them.
__global__ void gla_scan_kernel(GlaArgs a) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int tokens = a.q_start[seq + 1] - a.q_start[seq];
    if (tokens <= 0) return;
    const int segments = (tokens + a.segment - 1) / a.segment;
    const int cells = a.dim * a.vdim;
    const int cell = blockIdx.z * blockDim.x + threadIdx.x;
    if (cell >= cells) return;
    const int row = cell / a.vdim;
    float S = a.state[((size_t)a.state_slots[seq] * a.heads + head) * cells + cell];
    const size_t first = ((size_t)seq * a.max_segments) * a.heads + head;
    const size_t stride = a.heads;      // from one segment's index to the next's
    constexpr int AHEAD = 4;
    for (int k0 = 0; k0 < segments; k0 += AHEAD) {
        float local[AHEAD], decay[AHEAD];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const int k = k0 + u;
            const bool more = k + 1 < segments;
            const size_t index = first + (size_t)k * stride;
            local[u] = more ? a.segment_state[index * cells + cell] : 0.0f;
            decay[u] = more ? a.segment_decay[index * a.dim + row] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const int k = k0 + u;
            if (k < segments) {
                a.segment_state[(first + (size_t)k * stride) * cells + cell] = S;
                if (k + 1 < segments) S = fmaf(decay[u], S, local[u]);
            }
        }
    }
}

// Rows of S per thread: the smallest of 16, 32, 64, 128 with which the partitions that cover `dim` fit a block.
static int gla_rows_per_thread(int dim, int column_threads) {
    const int choices[4] = {16, 32, 64, 128};
    for (int c = 0; c < 4; ++c) {
        const int partitions = (dim + choices[c] - 1) / choices[c];
        // 128 rows of state per thread leave room for 256 threads' registers only
        if (partitions * column_threads <= (choices[c] == 128 ? 256 : 512)) return choices[c];
    }
    if ((dim + 127) / 128 * column_threads <= 512) return 129;      // 128 rows with 512 threads: the state spills
    return 0;
}

LLM_EXPORT int llm_gla_supports(int dim, int vdim) {
    if (dim <= 0 || vdim <= 0 || vdim > 512) return 0;
    return gla_rows_per_thread(dim, (vdim + 31) / 32 * 32) != 0;
}

LLM_EXPORT int llm_gla_recurrent(const void* proj, int row_width, int q_offset, int k_offset, int v_offset, int g_offset,
                                 const float* z, const float* z_bias, const void* weight, float* state, const int* state_slots,
                                 const int* q_start, void* out, int n_seqs, int heads, int dim, int vdim, float inverse_tau,
                                 float q_scale, float eps, int dtype, int weight_dtype, int segment, int max_segments,
                                 float* segment_state, float* segment_decay, cudaStream_t stream) {
    if (n_seqs == 0) return LLM_OK;
    if (!llm_gla_supports(dim, vdim) || heads <= 0) {
        llm_set_error("gla_recurrent: %d heads of %d key and %d value channels are not supported", heads, dim, vdim);
        return LLM_REFUSED;
    }
    GlaArgs a;
    a.proj = proj; a.row_width = row_width; a.q_offset = q_offset; a.k_offset = k_offset; a.v_offset = v_offset; a.g_offset = g_offset;
    a.z = z; a.z_bias = z_bias; a.weight = weight; a.state = state; a.state_slots = state_slots; a.q_start = q_start; a.out = out;
    a.heads = heads; a.dim = dim; a.vdim = vdim;
    a.column_threads = (vdim + 31) / 32 * 32;
    const int choice = gla_rows_per_thread(dim, a.column_threads);
    const int rows = choice == 129 ? 128 : choice;
    a.partitions = (dim + rows - 1) / rows;
    a.padded_dim = a.partitions * rows;
    a.inverse_tau = inverse_tau; a.q_scale = q_scale; a.eps = eps;
    a.segment = segment; a.max_segments = max_segments; a.segment_state = segment_state; a.segment_decay = segment_decay;
    const bool segmented = segment > 0;
    if (segmented && (max_segments <= 0 || !segment_state || !segment_decay)) {
        llm_set_error("gla_recurrent: the segmented form needs its scratch");
        return LLM_REFUSED;
    }
    const int threads = a.partitions * a.column_threads;
    const size_t shared = ((size_t)3 * GLA_TOKENS * a.padded_dim + (size_t)GLA_TOKENS * vdim + (size_t)a.partitions * GLA_TOKENS * vdim) * sizeof(float);
    dim3 grid(n_seqs, heads, segmented ? max_segments : 1);
#define GLA_LAUNCH_MODE(R, MODE)                                                                                        \
    do {                                                                                                                \
        if (shared > 40 * 1024) {                                                                                       \
            const int status = llm_raise_shared_limit((const void*)gla_recurrent_kernel<T, W, R, MODE>, shared, "gla_recurrent"); \
            if (status != LLM_OK) return status;                                                                        \
        }                                                                                                               \
        llm_launch(gla_recurrent_kernel<T, W, R, MODE>, grid, threads, shared, stream, a);                              \
    } while (0)
#define GLA_LAUNCH(R)                                                                                                   \
    do {                                                                                                                \
        if (!segmented) {                                                                                               \
            GLA_LAUNCH_MODE(R, GLA_ONE_PASS);                                                                           \
        } else {                                                                                                        \
            GLA_LAUNCH_MODE(R, GLA_LOCAL);                                                                              \
            llm_launch(gla_scan_kernel, dim3(n_seqs, heads, (dim * vdim + 255) / 256), 256, 0, stream, a);                            \
            GLA_LAUNCH_MODE(R, GLA_OUTPUT);                                                                             \
        }                                                                                                               \
    } while (0)
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, {
        if (choice == 16) GLA_LAUNCH(16);
        else if (choice == 32) GLA_LAUNCH(32);
        else if (choice == 64) GLA_LAUNCH(64);
        else if (choice == 128) GLA_LAUNCH(128);
        else GLA_LAUNCH(129);
    });
#undef GLA_LAUNCH
#undef GLA_LAUNCH_MODE
    return llm_check_launch("gla_recurrent");
}
