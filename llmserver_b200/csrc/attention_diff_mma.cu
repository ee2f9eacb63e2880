// Differential attention over the paged cache on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit
// accumulation): prompt portions and single decoded tokens in one launch.  The function is attention_diff.cu's:
//     s_m = cap(q_m . k_m * scale),  a_m = softmax(s_m) V  (m = 1, 2),  o = a_1 - lambda * a_2,
//     out = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)
//
// Rows of a tile are (token, head of the group) pairs of one sequence and one key/value head, so a decode step's tile
// is the group's heads of one token.  A warp owns 16 rows and ONE map: for a tile of 16 keys it forms S = Q_m K_m^T,
// updates its running maximum and sum and multiplies P V; the warp beside it does the same for the other map.  A block
// has 8 warps = row tiles x 2 maps x key splits: 2 x 2 x 2 for steps with prompt portions (measured ahead of 4 x 2 x 1
// and 1 x 2 x 4 at 2048 tokens with a window of 1024), 1 x 2 x 4 for steps of single tokens.  Every warp runs a pipeline of its own, cp.async into shared memory of its own, with no block barrier
// inside the key loop; with 128 registers a thread two blocks share an SM, which is what hides the latencies of
// ldmatrix, MMA and the exponentials (one warp with both maps needed 255 registers, one block per SM, and ran the
// tensor pipe at 23 %).  Attention weights stay 32-bit-grade through the P V product: each is carried as the sum of two
// bfloat16 numbers (its rounding and the rounding of the rest), two MMAs.  At the end the warps' partial results meet
// in shared memory; one warp per row merges the splits, subtracts the maps, normalises the head, applies the gate and
// stores.
//
// Sizes: units of 64 or 128 elements per map, values of 64 or 128; any group, window, page size (pages need not
// align with tiles: every key's page is looked up).  Other sizes run attention_diff.cu.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t shared_address(const void* pointer) { return (uint32_t)__cvta_generic_to_shared(pointer); }

__device__ __forceinline__ void copy_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void copy_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}
__device__ __forceinline__ void load_matrices(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void load_matrices_transposed(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void multiply_add(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_pair(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}
// What rounding (low, high) to the bfloat16 pair `packed` left over, itself rounded to bfloat16.
__device__ __forceinline__ uint32_t pack_rest(float low, float high, uint32_t packed) {
    const float2 rounded = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
    return pack_pair(low - rounded.x, high - rounded.y);
}

struct DiffParams {
    const __nv_bfloat16* q;
    int q_stride;
    const __nv_bfloat16* gate;     // null: no gate
    int gate_stride;
    const __nv_bfloat16* k_pages;  // [page, kv_head, slot, 2 * DIM]
    const __nv_bfloat16* v_pages;  // [page, kv_head, slot, DV]
    const int* block_tables;
    int max_blocks;
    const int* q_start;            // [S + 1]
    const int* context_len;        // [S]
    __nv_bfloat16* out;            // [N, heads * DV]
    int n_q_heads, n_kv_heads, page_size, num_pages;
    float scale, cap, lambda, eps, out_scale;
    int window, row_tiles;
    int* error_flag;
    int block_splits;              // single tokens only: blocks that share a (sequence, key/value head) pair's keys
    float* partials;               // [S, kv heads, block_splits * warp splits, 2 maps, group, DV + 2] when block_splits > 1
};

constexpr int kWarps = 8;
constexpr int kKeys = 16;    // keys per tile
constexpr int kPad = 8;      // elements of padding per shared-memory row: rows 16 bytes apart modulo 128, conflict-free ldmatrix

template <int DIM, int DV>
struct DiffShape {
    static constexpr int kKeyRow = DIM + kPad, kValueRow = DV + kPad;      // a warp holds its own map's half of a key row
    static constexpr int kQBytes = 16 * kKeyRow * 2, kKBytes = kKeys * kKeyRow * 2, kVBytes = kKeys * kValueRow * 2;
    static constexpr int kPartialBytes = 16 * DV * 4 + 16 * 2 * 4;         // a warp's O [16 rows][DV], then max and sum [16][2]
    static constexpr int kTileBytes = kQBytes + kKBytes + kVBytes;
    static constexpr int kWarpBytes = kTileBytes > kPartialBytes ? kTileBytes : kPartialBytes;
};

// 1 - 2 / (exp(2x) + 1): the hardware exponential and a fast division; absolute error of a few 1e-7, exact limits
__device__ __forceinline__ float fast_tanh(float x) { return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f); }

// Where key `key` of the sequence lies in the pages (in slots of one key/value head); keys behind the context read the
// last key, and are masked by their scores.
__device__ __forceinline__ long long slot_of_key(const DiffParams& p, const int* table, int key, int context, int kv_head) {
    key = min(key, context - 1);
    int page = table[key / p.page_size];
    if ((unsigned)page >= (unsigned)p.num_pages) {
        atomicExch(p.error_flag, 5);
        page = 0;
    }
    return ((long long)page * p.n_kv_heads + kv_head) * p.page_size + key % p.page_size;
}

template <int DIM, int DV>
__global__ void __launch_bounds__(kWarps * 32, 2) attention_diff_mma_kernel(DiffParams p) {
    pdl_trigger();
    pdl_wait();
    using Shape = DiffShape<DIM, DV>;
    constexpr int KT = kKeys;
    constexpr int kKeyChunks = DIM / 8, kValueChunks = DV / 8;
    extern __shared__ uint4 diff_shared_raw[];
    unsigned char* shared = reinterpret_cast<unsigned char*>(diff_shared_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sequence = blockIdx.y, kv_head = blockIdx.z % p.n_kv_heads, block_split = blockIdx.z / p.n_kv_heads;
    const int group = p.n_q_heads / p.n_kv_heads;
    const int begin = p.q_start[sequence], q_len = p.q_start[sequence + 1] - begin;
    const int context = p.context_len[sequence];
    const int start = context - q_len;                  // position of the portion's first token
    const int total_rows = q_len * group;
    const int row_tiles = p.row_tiles, splits = kWarps / (2 * row_tiles);
    const int block_row0 = blockIdx.x * 16 * row_tiles;
    if (block_row0 >= total_rows) return;
    // warp = tile + row_tiles * (map + 2 * split)
    const int tile = warp % row_tiles, map = (warp / row_tiles) & 1, split = warp / (2 * row_tiles);
    const int row0 = block_row0 + tile * 16;
    unsigned char* mine = shared + (size_t)warp * Shape::kWarpBytes;      // the warp's tiles, and its partial result at the end
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(mine);
    __nv_bfloat16* k_tile = reinterpret_cast<__nv_bfloat16*>(mine + Shape::kQBytes);
    __nv_bfloat16* v_tile = reinterpret_cast<__nv_bfloat16*>(mine + Shape::kQBytes + Shape::kKBytes);
    const int* table = p.block_tables + (size_t)sequence * p.max_blocks;
    const bool tile_live = row0 < total_rows;
    const float inverse_cap = p.cap > 0.0f ? 1.0f / p.cap : 0.0f;

    // this lane's two rows of the tile: the C-fragment rows lane / 4 and lane / 4 + 8
    int row_position[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = row0 + (lane >> 2) + 8 * h;
        row_position[h] = r < total_rows ? start + r / group : -1;      // -1: no such row, nothing is visible
    }
    float acc[DV / 8][4];
    float running_max[2] = {-INFINITY, -INFINITY}, running_sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    if (tile_live) {
        // the map's queries of the tile's 16 rows into the warp's shared memory (rows that do not exist: zeros)
        for (int c = lane; c < 16 * kKeyChunks; c += 32) {
            const int r = c / kKeyChunks, chunk = c % kKeyChunks, row = row0 + r;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (row < total_rows) {
                const int token = begin + row / group, head = kv_head * group + row % group;
                value = *reinterpret_cast<const uint4*>(p.q + (size_t)token * p.q_stride + ((size_t)head * 2 + map) * DIM + chunk * 8);
            }
            *reinterpret_cast<uint4*>(q_tile + r * Shape::kKeyRow + chunk * 8) = value;
        }
        // the keys this warp's rows see between them, and the keys every one of its rows sees
        const int last_row = min(row0 + 15, total_rows - 1);
        const int warp_first = start + row0 / group, warp_last = start + last_row / group;     // positions of its first and last row
        const int key_low = p.window > 0 ? max(0, warp_first - p.window + 1) : 0;
        const int key_high = warp_last;
        const int whole_low = p.window > 0 ? max(0, warp_last - p.window + 1) : 0, whole_high = warp_first;
        const int n_tiles = (key_high - key_low + KT) / KT;
        const int all_splits = splits * p.block_splits;
        const int per_split = (n_tiles + all_splits - 1) / all_splits;
        const int tile_begin = (block_split * splits + split) * per_split, tile_end = min(n_tiles, tile_begin + per_split);

        for (int t = tile_begin; t < tile_end; ++t) {
            const int key0 = key_low + t * KT;
            __syncwarp();      // everyone has read the tile before
            const long long slot = lane < KT ? slot_of_key(p, table, key0 + lane, context, kv_head) : 0;      // lane = key
#pragma unroll
            for (int c = lane; c < KT * kKeyChunks; c += 32) {
                const int key = c / kKeyChunks, chunk = c % kKeyChunks;
                const long long at = __shfl_sync(0xffffffffu, slot, key);
                copy_async_16(shared_address(k_tile + key * Shape::kKeyRow + chunk * 8), p.k_pages + (at * 2 + map) * DIM + chunk * 8);
            }
#pragma unroll
            for (int c = lane; c < KT * kValueChunks; c += 32) {
                const int key = c / kValueChunks, chunk = c % kValueChunks;
                const long long at = __shfl_sync(0xffffffffu, slot, key);
                copy_async_16(shared_address(v_tile + key * Shape::kValueRow + chunk * 8), p.v_pages + at * DV + chunk * 8);
            }
            copy_async_wait_all();
            __syncwarp();
            // every key of the tile is visible to every row of the warp: no score needs masking
            const bool whole = key0 >= whole_low && key0 + KT - 1 <= whole_high && row0 + 15 < total_rows;

            // S = Q_m K_m^T for 16 rows x KT keys
            float s[KT / 8][4];
#pragma unroll
            for (int j = 0; j < KT / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DIM / 16; ++ks) {
                uint32_t a[4], b[4];
                load_matrices(a, shared_address(q_tile + ((lane & 7) + 8 * ((lane >> 3) & 1)) * Shape::kKeyRow + ks * 16 + 8 * (lane >> 4)));
                load_matrices(b, shared_address(k_tile + ((lane & 7) + 8 * (lane >> 4)) * Shape::kKeyRow + ks * 16 + 8 * ((lane >> 3) & 1)));
                multiply_add(s[0], a, b[0], b[1]);
                multiply_add(s[1], a, b[2], b[3]);
            }
            // scale, cap, mask; the rows' maxima
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    float value = s[j][e] * p.scale;
                    if (p.cap > 0.0f) value = p.cap * fast_tanh(value * inverse_cap);
                    if (!whole) {
                        const int key = key0 + 8 * j + 2 * (lane & 3) + (e & 1);
                        const bool seen = key <= row_position[h] && (p.window <= 0 || key > row_position[h] - p.window);
                        value = seen ? value : -INFINITY;
                    }
                    s[j][e] = value;
                    tile_max[h] = fmaxf(tile_max[h], value);
                }
            }
            float correction[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
                tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
                const float new_max = fmaxf(running_max[h], tile_max[h]);
                // a row that has seen nothing yet keeps a maximum of -inf: subtract 0 there, its weights are exp(-inf) = 0
                const float safe_max = new_max == -INFINITY ? 0.0f : new_max;
                correction[h] = __expf(running_max[h] - safe_max);      // exp(-inf) = 0 on the first tile
                running_max[h] = new_max;
                tile_max[h] = safe_max;
            }
            float tile_sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float weight = __expf(s[j][e] - tile_max[e >> 1]);
                    s[j][e] = weight;
                    tile_sum[e >> 1] += weight;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tile_sum[h] += __shfl_xor_sync(0xffffffffu, tile_sum[h], 1);
                tile_sum[h] += __shfl_xor_sync(0xffffffffu, tile_sum[h], 2);
                running_sum[h] = running_sum[h] * correction[h] + tile_sum[h];
            }
            if (correction[0] != 1.0f || correction[1] != 1.0f) {     // a maximum moved
#pragma unroll
                for (int j = 0; j < DV / 8; ++j) {
                    acc[j][0] *= correction[0];
                    acc[j][1] *= correction[0];
                    acc[j][2] *= correction[1];
                    acc[j][3] *= correction[1];
                }
            }
            // O += P V with P as two bfloat16 parts (KT = 16 keys: one k-step)
            uint32_t high[4], low[4];
            high[0] = pack_pair(s[0][0], s[0][1]);
            high[1] = pack_pair(s[0][2], s[0][3]);
            high[2] = pack_pair(s[1][0], s[1][1]);
            high[3] = pack_pair(s[1][2], s[1][3]);
            low[0] = pack_rest(s[0][0], s[0][1], high[0]);
            low[1] = pack_rest(s[0][2], s[0][3], high[1]);
            low[2] = pack_rest(s[1][0], s[1][1], high[2]);
            low[3] = pack_rest(s[1][2], s[1][3], high[3]);
            // two column pairs at a time, the four MMAs of one part before those of the other: an accumulator's next
            // MMA comes four instructions after its last
#pragma unroll
            for (int jp = 0; jp < DV / 16; jp += 2) {
                uint32_t b[4], c[4];
                const int key_row = (lane & 7) + 8 * ((lane >> 3) & 1);
                load_matrices_transposed(b, shared_address(v_tile + key_row * Shape::kValueRow + jp * 16 + 8 * (lane >> 4)));
                load_matrices_transposed(c, shared_address(v_tile + key_row * Shape::kValueRow + (jp + 1) * 16 + 8 * (lane >> 4)));
                multiply_add(acc[2 * jp], high, b[0], b[1]);
                multiply_add(acc[2 * jp + 1], high, b[2], b[3]);
                multiply_add(acc[2 * jp + 2], high, c[0], c[1]);
                multiply_add(acc[2 * jp + 3], high, c[2], c[3]);
                multiply_add(acc[2 * jp], low, b[0], b[1]);
                multiply_add(acc[2 * jp + 1], low, b[2], b[3]);
                multiply_add(acc[2 * jp + 2], low, c[0], c[1]);
                multiply_add(acc[2 * jp + 3], low, c[2], c[3]);
            }
        }
        __syncwarp();
        if (p.block_splits > 1) {
            // several blocks share the keys: the warp's rows go to global memory, and a kernel of its own merges them
            const size_t slot = (((size_t)sequence * p.n_kv_heads + kv_head) * all_splits + block_split * splits + split) * 2 + map;
            float* rows = p.partials + slot * group * (DV + 2);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = row0 + (lane >> 2) + 8 * h;
                if (r < total_rows) {
#pragma unroll
                    for (int j = 0; j < DV / 8; ++j)
                        *reinterpret_cast<float2*>(rows + (size_t)r * (DV + 2) + 8 * j + 2 * (lane & 3)) = make_float2(acc[j][2 * h], acc[j][2 * h + 1]);
                    if ((lane & 3) == 0) *reinterpret_cast<float2*>(rows + (size_t)r * (DV + 2) + DV) = make_float2(running_max[h], running_sum[h]);
                }
            }
            return;
        }
        // the warp's partial result takes the place of its tiles: O [16 rows][DV], then max and sum [16][2]
        float* partial = reinterpret_cast<float*>(mine);
        float* statistics = partial + 16 * DV;
#pragma unroll
        for (int j = 0; j < DV / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = (lane >> 2) + 8 * (e >> 1), column = 8 * j + 2 * (lane & 3) + (e & 1);
                partial[r * DV + column] = acc[j][e];
            }
        }
        if ((lane & 3) == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = (lane >> 2) + 8 * h;
                statistics[r * 2] = running_max[h];
                statistics[r * 2 + 1] = running_sum[h];
            }
        }
    }
    if (p.block_splits > 1) return;      // (uniform over the block)
    __syncthreads();
    // one warp per row: merge the splits of each map, subtract the maps, normalise the head, gate, store
    const int block_rows = min(16 * row_tiles, total_rows - block_row0);
    for (int r = warp; r < block_rows; r += kWarps) {
        const int in_tile = r % 16, which_tile = r / 16;
        float merged[2][DV / 32];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float top = -INFINITY;
            for (int s = 0; s < splits; ++s) {
                const float* statistics = reinterpret_cast<const float*>(shared + (size_t)(which_tile + row_tiles * (m + 2 * s)) * Shape::kWarpBytes) + 16 * DV;
                top = fmaxf(top, statistics[in_tile * 2]);
            }
            float denominator = 0.0f;
#pragma unroll
            for (int i = 0; i < DV / 32; ++i) merged[m][i] = 0.0f;
            for (int s = 0; s < splits; ++s) {
                const float* partial = reinterpret_cast<const float*>(shared + (size_t)(which_tile + row_tiles * (m + 2 * s)) * Shape::kWarpBytes);
                const float* statistics = partial + 16 * DV;
                const float own_max = statistics[in_tile * 2];
                if (own_max == -INFINITY) continue;          // this split saw no key of the row
                const float factor = __expf(own_max - top);
                denominator += factor * statistics[in_tile * 2 + 1];
#pragma unroll
                for (int i = 0; i < DV / 32; ++i) merged[m][i] += factor * partial[in_tile * DV + lane + 32 * i];
            }
            const float inverse = 1.0f / denominator;
#pragma unroll
            for (int i = 0; i < DV / 32; ++i) merged[m][i] *= inverse;
        }
        float sum_squares = 0.0f;
#pragma unroll
        for (int i = 0; i < DV / 32; ++i) {
            merged[0][i] -= p.lambda * merged[1][i];
            sum_squares += merged[0][i] * merged[0][i];
        }
        const int row = block_row0 + r;
        const int token = begin + row / group, head = kv_head * group + row % group;
        float factor = rsqrtf(warp_sum(sum_squares) / (float)DV + p.eps) * p.out_scale;
        if (p.gate) {
            const float g = __bfloat162float(p.gate[(size_t)token * p.gate_stride + head]);
            factor *= 1.0f / (1.0f + __expf(-g));
        }
        __nv_bfloat16* dst = p.out + (size_t)token * p.n_q_heads * DV + (size_t)head * DV;
#pragma unroll
        for (int i = 0; i < DV / 32; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(merged[0][i] * factor);
    }
}

// Single tokens whose keys several blocks shared: one warp per (sequence, head) merges the partial results of all
// splits for each map, subtracts the maps, normalises the head, applies the gate and stores.
template <int DV>
__global__ void attention_diff_merge_kernel(DiffParams p, int all_splits) {
    pdl_trigger();
    pdl_wait();
    const int sequence = blockIdx.x, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (head >= p.n_q_heads) return;
    const int group = p.n_q_heads / p.n_kv_heads;
    const int kv_head = head / group, r = head % group;
    const int token = p.q_start[sequence];
    if (p.q_start[sequence + 1] - token != 1) return;      // this launch shape is for single tokens only
    const float* base = p.partials + ((size_t)sequence * p.n_kv_heads + kv_head) * all_splits * 2 * group * (DV + 2);
    float merged[2][DV / 32];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        // lanes own the splits' maxima and sums (at most 64 splits), so these loads do not wait for one another
        float own_max[2], own_sum[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int s = lane + 32 * u;
            float2 statistics = make_float2(-INFINITY, 0.0f);
            if (s < all_splits) statistics = *reinterpret_cast<const float2*>(base + ((size_t)(s * 2 + m) * group + r) * (DV + 2) + DV);
            own_max[u] = statistics.x;
            own_sum[u] = statistics.y;
        }
        const float top = warp_max(fmaxf(own_max[0], own_max[1]));
        float factor[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) factor[u] = own_max[u] == -INFINITY ? 0.0f : __expf(own_max[u] - top);      // a split that saw no key
        const float inverse = 1.0f / warp_sum(factor[0] * own_sum[0] + factor[1] * own_sum[1]);
#pragma unroll
        for (int i = 0; i < DV / 32; ++i) merged[m][i] = 0.0f;
#pragma unroll 4
        for (int s = 0; s < all_splits; ++s) {
            const float f = __shfl_sync(0xffffffffu, s < 32 ? factor[0] : factor[1], s & 31);
            const float* row = base + ((size_t)(s * 2 + m) * group + r) * (DV + 2);
#pragma unroll
            for (int i = 0; i < DV / 32; ++i) merged[m][i] = fmaf(f, row[lane + 32 * i], merged[m][i]);
        }
#pragma unroll
        for (int i = 0; i < DV / 32; ++i) merged[m][i] *= inverse;
    }
    float sum_squares = 0.0f;
#pragma unroll
    for (int i = 0; i < DV / 32; ++i) {
        merged[0][i] -= p.lambda * merged[1][i];
        sum_squares += merged[0][i] * merged[0][i];
    }
    float factor = rsqrtf(warp_sum(sum_squares) / (float)DV + p.eps) * p.out_scale;
    if (p.gate) {
        const float g = __bfloat162float(p.gate[(size_t)token * p.gate_stride + head]);
        factor *= 1.0f / (1.0f + __expf(-g));
    }
    __nv_bfloat16* dst = p.out + (size_t)token * p.n_q_heads * DV + (size_t)head * DV;
#pragma unroll
    for (int i = 0; i < DV / 32; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(merged[0][i] * factor);
}

template <int DIM, int DV>
int launch_diff(const DiffParams& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    using Shape = DiffShape<DIM, DV>;
    const size_t shared = (size_t)kWarps * Shape::kWarpBytes;
    const int status = llm_raise_shared_limit((const void*)attention_diff_mma_kernel<DIM, DV>, shared, "attention_diff_mma");
    if (status != LLM_OK) return status;
    const int group = p.n_q_heads / p.n_kv_heads;
    const int rows = max_q_len * group;
    dim3 grid((rows + 16 * p.row_tiles - 1) / (16 * p.row_tiles), n_seqs, p.n_kv_heads * p.block_splits);
    llm_launch(attention_diff_mma_kernel<DIM, DV>, grid, kWarps * 32, shared, stream, p);
    if (p.block_splits > 1) {
        const int all_splits = p.block_splits * (kWarps / (2 * p.row_tiles));
        llm_launch(attention_diff_merge_kernel<DV>, dim3(n_seqs, (p.n_q_heads + 3) / 4), 128, 0, stream, p, all_splits);
    }
    return llm_check_launch("attention_diff_mma");
}

}  // namespace

LLM_EXPORT int llm_attention_diff_mma_supports(int dim, int value_dim, int n_q_heads, int n_kv_heads) {
    return (dim == 64 || dim == 128) && (value_dim == 64 || value_dim == 128) && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0;
}

LLM_EXPORT int llm_attention_diff_mma(const void* q, int q_stride, const void* gate, int gate_stride, const void* k_pages,
                                      const void* v_pages, const int* block_tables, int max_blocks, const int* q_start,
                                      const int* context_len, void* out, int n_seqs, int max_q_len, int n_q_heads, int n_kv_heads,
                                      int dim, int value_dim, int page_size, int num_pages, float scale, float cap, int window,
                                      float lambda, float eps, float out_scale, int* error_flag, int row_tiles, int block_splits,
                                      float* partials, cudaStream_t stream) {
    if (n_seqs == 0 || max_q_len == 0) return LLM_OK;
    if (!llm_attention_diff_mma_supports(dim, value_dim, n_q_heads, n_kv_heads) || page_size <= 0 || num_pages <= 0) {
        llm_set_error("attention_diff_mma: units of %d, values of %d, %d / %d heads are not supported", dim, value_dim, n_q_heads, n_kv_heads);
        return LLM_REFUSED;
    }
    if (q_stride % 8 || !aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages)) {
        llm_set_error("attention_diff_mma: queries and pages must be 16-byte aligned (query stride %d)", q_stride);
        return LLM_REFUSED;
    }
    DiffParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.gate = (const __nv_bfloat16*)gate; p.gate_stride = gate_stride;
    p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages; p.block_tables = block_tables;
    p.max_blocks = max_blocks; p.q_start = q_start; p.context_len = context_len; p.out = (__nv_bfloat16*)out;
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.num_pages = num_pages;
    p.scale = scale; p.cap = cap; p.lambda = lambda; p.eps = eps; p.out_scale = out_scale; p.window = window;
    // 8: the warps share their key tiles (prompt portions); 1, 2, 4: the rest of the warps split a tile's keys
    // 2 row tiles (and 2 key splits) for steps with prompt portions, 1 (and 4 key splits) for steps of single tokens
    p.row_tiles = (row_tiles == 1 || row_tiles == 2 || row_tiles == 4) ? row_tiles : (max_q_len > 1 ? 2 : 1);
    p.error_flag = error_flag;
    // several blocks per (sequence, key/value head) pair only for steps of single tokens whose group fits one row tile
    p.block_splits = (max_q_len == 1 && p.row_tiles == 1 && n_q_heads / n_kv_heads <= 16 && partials && block_splits > 1) ? block_splits : 1;
    p.partials = partials;
    if (dim == 64 && value_dim == 64) return launch_diff<64, 64>(p, n_seqs, max_q_len, stream);
    if (dim == 64 && value_dim == 128) return launch_diff<64, 128>(p, n_seqs, max_q_len, stream);
    if (dim == 128 && value_dim == 64) return launch_diff<128, 64>(p, n_seqs, max_q_len, stream);
    return launch_diff<128, 128>(p, n_seqs, max_q_len, stream);
}
