// Latent attention: every token leaves one row [latent | rope] in its request's pages (the normed latent
// vector and one rotated key part shared by all heads).  A query head is given in the latent's space,
// [W_uk_h^T q_plain_h | rope(q_rot_h)], so that its score against a cached row is one dot product and the
// weighted sum of the rows' latent parts is what the head's value projection is applied to afterwards.
//
//   latent_prepare           norm of the latent, rotation of the shared key part and of the queries' rotated parts,
//                            the page write, and the queries laid out [token][head][latent | rope]
//   latent_attention_plain   one block per (token, head): 32-bit scores, softmax and sums; the 32-bit path's
//                            attention and the reference for the tensor-core kernel
//   gate_heads               heads' values [head][token][vdim] times sigmoid(gate), laid out [token][head * vdim]
#include "common.cuh"

namespace lb {

struct LatentLayout {
    int page_size;
    int num_pages;
    int max_blocks;   // columns of the block table
    int latent;       // channels of the normed latent vector (also the value a row stands for)
    int rope;         // channels of the rotated key part
};

template <typename T>
__device__ __forceinline__ T* latent_row(T* pages, const int* block_table, const LatentLayout& layout, int segment, int position) {
    const int block = position / layout.page_size;
    if (block >= layout.max_blocks) return nullptr;
    const int page = block_table[static_cast<size_t>(segment) * layout.max_blocks + block];
    if (page < 0 || page >= layout.num_pages) return nullptr;
    const size_t row = static_cast<size_t>(page) * layout.page_size + (position - block * layout.page_size);
    return pages + row * (layout.latent + layout.rope);
}

// One block per token.
//   q        [tokens][q_stride]: head h at h * (head_dim + rope), its last `rope` channels are rotated
//   q_latent [heads][tokens][latent]: the heads' unrotated parts taken into the latent's space
//   down     [tokens][down_stride]: [latent | rope]
//   q_out    [tokens][heads][latent + rope]
//   pages    [page][row][latent + rope]: row = [T(norm(down[:latent]) * (w + offset)) | rope(down[latent:])]
// The rotation pairs channel i with i + rope / 2: (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * inv_freq[i].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ q_latent, const T* __restrict__ down, int down_stride,
                                      T* __restrict__ q_out, T* __restrict__ pages, const float* __restrict__ norm_weight, float eps, float scale_offset,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions, const int* __restrict__ token_segment,
                                      const int* __restrict__ block_table, LatentLayout layout, int tokens, int num_heads, int head_dim, int write_kv,
                                      int* status) {
    extern __shared__ float shared[];
    const int half = layout.rope / 2, latent = layout.latent, rope = layout.rope;
    float* cosines = shared;            // half
    float* sines = shared + half;       // half
    float* scratch = sines + half;      // 33
    const int token = blockIdx.x;
    const int position = positions[token];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(static_cast<float>(position) * inv_freq[i], &sines[i], &cosines[i]);
    const T* row = down + static_cast<size_t>(token) * down_stride;
    float squares = 0.0f;
    if (write_kv) {
        for (int d = threadIdx.x; d < latent; d += blockDim.x) {
            const float v = to_float(row[d]);
            squares += v * v;
        }
    }
    const float total = block_sum(squares, scratch);   // also orders the writes to cosines[] and sines[]
    if (write_kv) {
        T* dst = latent_row(pages, block_table, layout, token_segment[token], position);
        if (dst == nullptr) {
            if (threadIdx.x == 0) report_error(status, kBadPage);
        } else {
            const float inv = rsqrtf(total / static_cast<float>(latent) + eps);
            for (int d = threadIdx.x; d < latent; d += blockDim.x) dst[d] = from_float<T>(to_float(row[d]) * inv * (norm_weight[d] + scale_offset));
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float u = to_float(row[latent + i]), v = to_float(row[latent + half + i]);
                dst[latent + i] = from_float<T>(u * cosines[i] - v * sines[i]);
                dst[latent + half + i] = from_float<T>(v * cosines[i] + u * sines[i]);
            }
        }
    }
    const int full = latent + rope;
    for (int head = 0; head < num_heads; ++head) {
        const T* q_head = q + static_cast<size_t>(token) * q_stride + static_cast<size_t>(head) * (head_dim + rope) + head_dim;
        const T* from = q_latent + (static_cast<size_t>(head) * tokens + token) * latent;
        T* to = q_out + (static_cast<size_t>(token) * num_heads + head) * full;
        for (int d = threadIdx.x; d < latent; d += blockDim.x) to[d] = from[d];
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = to_float(q_head[i]), v = to_float(q_head[half + i]);
            to[latent + i] = from_float<T>(u * cosines[i] - v * sines[i]);
            to[latent + half + i] = from_float<T>(v * cosines[i] + u * sines[i]);
        }
    }
}

constexpr int kLatentThreads = 128, kLatentChunk = 128, kLatentMaxDimsPerThread = 8;   // latent <= 1024

// grid (tokens, heads).  The query at position p sees the rows j with max(0, p - window + 1) <= j <= p (window <= 0:
// all j <= p).  Rows are visited in chunks that start at the first visible row, so the result does not depend on how a
// prompt was cut into steps or on what else is in the batch.  out [tokens][heads][latent].
template <typename T>
__global__ void latent_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pages, T* __restrict__ out, const int* __restrict__ positions,
                                              const int* __restrict__ token_segment, const int* __restrict__ block_table, LatentLayout layout, int num_heads,
                                              float scale, int window, int* status) {
    extern __shared__ __align__(16) float shared[];
    const int latent = layout.latent, full = layout.latent + layout.rope;
    const T** rows = reinterpret_cast<const T**>(shared);                       // kLatentChunk pointers
    float* scores = shared + 2 * kLatentChunk;                                   // kLatentChunk
    float* scratch = scores + kLatentChunk;                                      // 33 (+ 3 to keep q_shared apart)
    float* q_shared = scratch + 36;                                              // full
    const int token = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int segment = token_segment[token];
    const int position = positions[token];
    const int first = window > 0 ? max(0, position - window + 1) : 0;
    const T* q_row = q + (static_cast<size_t>(token) * num_heads + head) * full;
    for (int d = tid; d < full; d += blockDim.x) q_shared[d] = to_float(q_row[d]);
    __syncthreads();

    float acc[kLatentMaxDimsPerThread];
#pragma unroll
    for (int i = 0; i < kLatentMaxDimsPerThread; ++i) acc[i] = 0.0f;
    float running_max = -INFINITY, running_sum = 0.0f;
    for (int chunk = first; chunk <= position; chunk += kLatentChunk) {
        const int count = min(kLatentChunk, position + 1 - chunk);
        float local_max = -INFINITY;
        for (int i = warp; i < count; i += kLatentThreads / 32) {   // a warp per row, lanes along its channels
            const T* row = latent_row(const_cast<T*>(pages), block_table, layout, segment, chunk + i);
            float s = -INFINITY;
            if (row == nullptr) {
                if (lane == 0) report_error(status, kBadPage);
            } else {
                float dot = 0.0f;
                for (int d = lane; d < full; d += 32) dot += q_shared[d] * to_float(row[d]);
                s = warp_sum(dot) * scale;
            }
            if (lane == 0) {
                rows[i] = row;
                scores[i] = s;
            }
            local_max = fmaxf(local_max, s);
        }
        const float chunk_max = block_max(local_max, scratch);
        const float new_max = fmaxf(running_max, chunk_max);
        const float rescale = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
        float local_sum = 0.0f;
        for (int i = tid; i < count; i += blockDim.x) {
            const float p = new_max == -INFINITY || rows[i] == nullptr ? 0.0f : expf(scores[i] - new_max);
            scores[i] = p;
            local_sum += p;
        }
        const float chunk_sum = block_sum(local_sum, scratch);   // also orders the writes to scores[]
        running_sum = running_sum * rescale + chunk_sum;
        running_max = new_max;
#pragma unroll
        for (int slot = 0; slot < kLatentMaxDimsPerThread; ++slot) {
            const int d = tid + slot * kLatentThreads;
            if (d < latent) {
                float sum = acc[slot] * rescale;
                for (int i = 0; i < count; ++i) {
                    const float p = scores[i];
                    if (p != 0.0f) sum += p * to_float(rows[i][d]);
                }
                acc[slot] = sum;
            }
        }
        __syncthreads();   // scores[] and rows[] are rewritten by the next chunk
    }
    T* dst = out + (static_cast<size_t>(token) * num_heads + head) * latent;
    const float norm = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
#pragma unroll
    for (int slot = 0; slot < kLatentMaxDimsPerThread; ++slot) {
        const int d = tid + slot * kLatentThreads;
        if (d < latent) dst[d] = from_float<T>(acc[slot] * norm);
    }
}

// out[t][h * vdim + j] = T(values[h][t][j] * sigmoid(gate[t * gate_stride + h * vdim + j]))   (gate null: no gate)
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ values, const T* __restrict__ gate, int gate_stride, T* __restrict__ out, int tokens, int num_heads,
                                  int value_dim) {
    const int token = blockIdx.x, width = num_heads * value_dim;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const int head = c / value_dim, j = c - head * value_dim;
        float v = to_float(values[(static_cast<size_t>(head) * tokens + token) * value_dim + j]);
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-to_float(gate[static_cast<size_t>(token) * gate_stride + c])));
        out[static_cast<size_t>(token) * width + c] = from_float<T>(v);
    }
}

}  // namespace lb

extern "C" {

int lb_latent_prepare(const void* q, int q_stride, const void* q_latent, const void* down, int down_stride, void* q_out, void* pages,
                      const float* norm_weight, float eps, float scale_offset, const float* inv_freq, const int* positions, const int* token_segment,
                      const int* block_table, int tokens, int num_heads, int head_dim, int latent, int rope, int page_size, int num_pages, int max_blocks,
                      int write_kv, int dtype, int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (rope < 0 || rope % 2 != 0 || latent < 1 || num_heads < 1) return -2;
    lb::LatentLayout layout{page_size, num_pages, max_blocks, latent, rope};
    const size_t shared = (static_cast<size_t>(rope) + 33) * sizeof(float);
    if (shared > 48 * 1024) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        lb::latent_prepare_kernel<T><<<tokens, 128, shared, stream>>>(
            static_cast<const T*>(q), q_stride, static_cast<const T*>(q_latent), static_cast<const T*>(down), down_stride, static_cast<T*>(q_out),
            static_cast<T*>(pages), norm_weight, eps, scale_offset, inv_freq, positions, token_segment, block_table, layout, tokens, num_heads, head_dim,
            write_kv, status);
    })
    return LB_LAUNCH_RESULT();
}

int lb_latent_attention_plain(const void* q, const void* pages, void* out, const int* positions, const int* token_segment, const int* block_table,
                              int tokens, int num_heads, int latent, int rope, int page_size, int num_pages, int max_blocks, float scale, int window,
                              int dtype, int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (latent < 1 || latent > lb::kLatentThreads * lb::kLatentMaxDimsPerThread || rope < 0) return -2;
    lb::LatentLayout layout{page_size, num_pages, max_blocks, latent, rope};
    const size_t shared = (3 * static_cast<size_t>(lb::kLatentChunk) + 36 + latent + rope) * sizeof(float);
    if (shared > 48 * 1024) return -2;
    const dim3 grid(tokens, num_heads);
    LB_DISPATCH_DTYPE(dtype, {
        lb::latent_attention_plain_kernel<T><<<grid, lb::kLatentThreads, shared, stream>>>(
            static_cast<const T*>(q), static_cast<const T*>(pages), static_cast<T*>(out), positions, token_segment, block_table, layout, num_heads, scale,
            window, status);
    })
    return LB_LAUNCH_RESULT();
}

int lb_gate_heads(const void* values, const void* gate, int gate_stride, void* out, int tokens, int num_heads, int value_dim, int dtype,
                  cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::gate_heads_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(values), static_cast<const T*>(gate), gate_stride, static_cast<T*>(out),
                                                              tokens, num_heads, value_dim);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
