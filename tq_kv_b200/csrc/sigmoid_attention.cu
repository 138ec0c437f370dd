// Attention whose weights are sigmoids instead of a softmax: the weight of a visible key j for the query at
// position i of head h is
//     sigmoid(q_i . k_j * scale + bias[h, min(i - j, n_dist - 1)])
// and the weights are not normalised over the keys: out_i = sum_j weight_ij * v_j, causal (j <= i).  `bias` is
// a float32 table per head and distance that the caller builds (a learned distance table looked up through
// its buckets, plus a constant per head); without a table the bias is zero.  The result of head h may be
// multiplied by sigmoid(gate[t, h]) (float32 logits, one per token and head).  Keys and values may differ in
// width (dk, dv), query heads share key/value heads in consecutive groups.
//
// Since nothing is normalised, partial sums over disjoint key ranges simply add: a long key range is cut into
// splits whose float32 partial results a second kernel adds in index order.
//
// The first kernel of this file prepares the operands: q and k rows are each divided by the root mean square
// of the WHOLE row (all heads together) and multiplied by a weight per entry, q is multiplied by a factor that
// grows with the logarithm of its position, and k and v are appended to the paged cache.
#include "common.cuh"

#define SA_MAX_COLS 8     // dv <= 256: each lane owns up to 8 value channels

struct SigKV {
    const void* k_packed;   // [T, nkv*dk] rows of this step (every sequence then starts at position 0)
    const void* v_packed;   // [T, nkv*dv]
    const void* k_pages;    // [pages, nkv, page_tokens, dk]
    const void* v_pages;    // [pages, nkv, page_tokens, dv]
    const int* block_table;
    int table_width;
    int page_tokens;
};

// ---------------------------------------------------------------------------
// Whole-row RMS norm of q and of k, the query's position factor, head split, cache append.
// x: [T, ldx] float32, columns [q (nh*dk) | k (nkv*dk) | v (nkv*dv) | ...]; biases were added by the product.
//   q_out = q / rms(q) * wq * (1 + coef * ln((pos + 1) / every + 1))     (integer division)
//   k     = k / rms(k) * wk
// Without wq / wk the rows pass unchanged; coef = 0 switches the factor off.  Rows at or past their sequence's
// new length are padding and are not cached.  One block per token.
// ---------------------------------------------------------------------------
template <typename TC>
__global__ void rownorm_qkv_store_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ wq,
                                         const float* __restrict__ wk, float eps, float coef, int every,
                                         const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                         const int* __restrict__ new_lens, const int* __restrict__ block_table,
                                         int table_width, int page_tokens, TC* __restrict__ q_out,
                                         TC* __restrict__ k_out, TC* __restrict__ v_out, TC* __restrict__ k_pages,
                                         TC* __restrict__ v_pages, int nh, int nkv, int dk, int dv) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int pos = tok_pos[t], b = tok_seq[t];
    const int nq = nh * dk, nk = nkv * dk, nv = nkv * dv;
    pdl_wait();
    pdl_launch();
    const float* xq = x + (size_t)t * ldx;
    const float* xk = xq + nq;
    const float* xv = xk + nk;
    float inv_q = 1.f, inv_k = 1.f;
    if (wq) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) ss = fmaf(xq[i], xq[i], ss);
        ss = block_sum(ss, red);
        inv_q = 1.f / sqrtf(ss / (float)nq + eps);
    }
    if (wk) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) ss = fmaf(xk[i], xk[i], ss);
        ss = block_sum(ss, red);
        inv_k = 1.f / sqrtf(ss / (float)nk + eps);
    }
    const float factor = coef != 0.f ? 1.f + coef * logf((float)((pos + 1) / every + 1)) : 1.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        float v = xq[i] * inv_q;
        if (wq) v *= wq[i];
        q_out[(size_t)t * nq + i] = from_f32<TC>(v * factor);
    }
    size_t page_row = 0;
    const bool to_cache = k_pages != nullptr && pos < new_lens[b];
    if (to_cache)
        page_row = (size_t)block_table[(size_t)b * table_width + pos / page_tokens] * nkv * page_tokens
                   + (pos % page_tokens);
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        float v = xk[i] * inv_k;
        if (wk) v *= wk[i];
        const TC r = from_f32<TC>(v);
        if (k_out) k_out[(size_t)t * nk + i] = r;
        if (to_cache) {
            const int g = i / dk, c = i - g * dk;
            k_pages[(page_row + (size_t)g * page_tokens) * dk + c] = r;
        }
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const TC r = from_f32<TC>(xv[i]);
        if (v_out) v_out[(size_t)t * nv + i] = r;
        if (to_cache) {
            const int g = i / dv, c = i - g * dv;
            v_pages[(page_row + (size_t)g * page_tokens) * dv + c] = r;
        }
    }
}

TQ_API int tq_rownorm_qkv_store(const float* x, int ldx, const float* wq, const float* wk, float eps, float coef,
                                int every, const int* tok_pos, const int* tok_seq, const int* new_lens,
                                const int* block_table, int table_width, int page_tokens, void* q_out, void* k_out,
                                void* v_out, void* k_pages, void* v_pages, int dtype, int n_tokens, int nh, int nkv,
                                int dk, int dv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!x || !q_out || nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || every <= 0) return (int)cudaErrorInvalidValue;
    if (k_pages && (!v_pages || !block_table || page_tokens <= 0 || !new_lens)) return (int)cudaErrorInvalidValue;
    const int threads = nh * dk >= 2048 ? 512 : 256;
#define TQ_LAUNCH(T)                                                                                               \
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, rownorm_qkv_store_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, x, \
                         ldx, wq, wk, eps, coef, every, tok_pos, tok_seq, new_lens, block_table, table_width,       \
                         page_tokens, (T*)q_out, (T*)k_out, (T*)v_out, (T*)k_pages, (T*)v_pages, nh, nkv, dk, dv)
    if (dtype == TQ_F32) TQ_LAUNCH(float);
    if (dtype == TQ_BF16) TQ_LAUNCH(bf16);
#undef TQ_LAUNCH
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// The general kernel (any widths up to 256, either precision, packed or paged keys).
// grid (token, kv head, split); warp w of a block serves query heads g*n_rep + w, + n_warps, ...; the lanes of a
// warp take 32 keys at a time (one dot product each), then the warp adds weight * value row by row, every lane
// owning value channels lane, lane + 32, ...
// ---------------------------------------------------------------------------
template <typename TC>
__device__ __forceinline__ void sig_rows(const SigKV& src, int b, int j, int g, int nkv, int dk, int dv, int tok0,
                                         const TC*& krow, const TC*& vrow) {
    if (src.k_packed) {
        const size_t r = (size_t)(tok0 + j) * nkv + g;
        krow = (const TC*)src.k_packed + r * dk;
        vrow = (const TC*)src.v_packed + r * dv;
    } else {
        const int page = src.block_table[(size_t)b * src.table_width + j / src.page_tokens];
        const size_t r = ((size_t)page * nkv + g) * src.page_tokens + (j % src.page_tokens);
        krow = (const TC*)src.k_pages + r * dk;
        vrow = (const TC*)src.v_pages + r * dv;
    }
}

template <typename TC>
__global__ void sigmoid_attention_kernel(const TC* __restrict__ q, SigKV src, const int* __restrict__ tok_pos,
                                         const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ start_pos, float scale,
                                         const float* __restrict__ bias, int n_dist, const float* __restrict__ gate,
                                         int ldg, TC* __restrict__ out, float* __restrict__ part, int nh, int nkv,
                                         int dk, int dv, int n_splits) {
    extern __shared__ float q_sh[];   // [n_warps][dk]
    const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int n_rep = nh / nkv;
    const int pos = tok_pos[t];
    const int b = tok_seq[t];
    const int tok0 = src.k_packed ? cu_seqlens[b] - start_pos[b] : 0;
    int lo = 0, hi = pos + 1;
    if (n_splits > 1) {
        const int split_len = (((pos + n_splits) / n_splits) + 31) & ~31;
        lo = split * split_len;
        if (lo + split_len < hi) hi = lo + split_len;
    }
    float* qs = q_sh + warp * dk;
    constexpr int VEC = Vec16<TC>::N;
    const bool vec = (dk % VEC) == 0;
    pdl_wait();
    pdl_launch();

    for (int hr = warp; hr < n_rep; hr += n_warps) {
        const int h = g * n_rep + hr;
        const TC* qrow = q + ((size_t)t * nh + h) * dk;
        const float* hb = bias ? bias + (size_t)h * n_dist : nullptr;
        __syncwarp();
        for (int c = lane; c < dk; c += 32) qs[c] = to_f32<TC>(qrow[c]);
        __syncwarp();
        float acc[SA_MAX_COLS];
#pragma unroll
        for (int i = 0; i < SA_MAX_COLS; ++i) acc[i] = 0.f;

        for (int base = lo; base < hi; base += 32) {
            const int j = base + lane;
            const bool valid = j < hi;
            const TC *krow = nullptr, *vrow = nullptr;
            float p = 0.f;
            if (valid) {
                sig_rows<TC>(src, b, j, g, nkv, dk, dv, tok0, krow, vrow);
                float dot = 0.f;
                if (vec) {
                    for (int c = 0; c < dk; c += VEC) {
                        float kv[VEC];
                        load16_f32<TC>(krow + c, kv);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) dot = fmaf(qs[c + e], kv[e], dot);
                    }
                } else {
                    for (int c = 0; c < dk; ++c) dot = fmaf(qs[c], to_f32<TC>(krow[c]), dot);
                }
                float s = dot * scale;
                if (hb) s += hb[min(pos - j, n_dist - 1)];
                p = 1.f / (1.f + expf(-s));
            }
            const int n_here = min(32, hi - base);
            for (int jj = 0; jj < n_here; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const TC* vr = (const TC*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
#pragma unroll
                for (int i = 0; i < SA_MAX_COLS; ++i) {
                    const int c = lane + 32 * i;
                    if (c < dv) acc[i] = fmaf(pj, to_f32<TC>(vr[c]), acc[i]);
                }
            }
        }
        if (n_splits == 1) {
            const float gt = gate ? 1.f / (1.f + expf(-gate[(size_t)t * ldg + h])) : 1.f;
            TC* o = out + ((size_t)t * nh + h) * dv;
#pragma unroll
            for (int i = 0; i < SA_MAX_COLS; ++i) {
                const int c = lane + 32 * i;
                if (c < dv) o[c] = from_f32<TC>(acc[i] * gt);
            }
        } else {
            float* pa = part + (((size_t)t * nh + h) * n_splits + split) * dv;
#pragma unroll
            for (int i = 0; i < SA_MAX_COLS; ++i) {
                const int c = lane + 32 * i;
                if (c < dv) pa[c] = acc[i];
            }
        }
    }
}

// Adds the splits of one (token, head) in index order and applies the gate.  grid (token, head).
template <typename TC>
__global__ void sigmoid_attention_sum_kernel(const float* __restrict__ part, const float* __restrict__ gate, int ldg,
                                             TC* __restrict__ out, int nh, int dv, int n_splits) {
    const int t = blockIdx.x, h = blockIdx.y;
    pdl_wait();
    pdl_launch();
    const float* pa = part + ((size_t)t * nh + h) * n_splits * dv;
    const float gt = gate ? 1.f / (1.f + expf(-gate[(size_t)t * ldg + h])) : 1.f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) a += pa[(size_t)s * dv + c];
        out[((size_t)t * nh + h) * dv + c] = from_f32<TC>(a * gt);
    }
}

// Scratch for n_splits > 1: float[T * nh * n_splits * dv].
TQ_API int tq_sigmoid_attention(const void* q, int dtype, const void* k_packed, const void* v_packed,
                                const void* k_pages, const void* v_pages, const int* block_table, int table_width,
                                int page_tokens, const int* tok_pos, const int* tok_seq, const int* cu_seqlens,
                                const int* start_pos, float scale, const float* bias, int n_dist, const float* gate,
                                int ldg, void* out, float* part, int n_tokens, int nh, int nkv, int dk, int dv,
                                int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || dv > 32 * SA_MAX_COLS || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
    if (n_splits < 1 || (n_splits > 1 && !part)) return (int)cudaErrorInvalidValue;
    if (!k_packed && (!k_pages || !block_table || page_tokens <= 0)) return (int)cudaErrorInvalidValue;
    if (nkv > 65535 || n_splits > 65535 || (bias && n_dist <= 0)) return (int)cudaErrorInvalidValue;
    SigKV src{k_packed, v_packed, k_pages, v_pages, block_table, table_width, page_tokens};
    const int n_rep = nh / nkv;
    const int n_warps = n_rep < 8 ? n_rep : 8;
    const dim3 grid(n_tokens, nkv, n_splits);
    const size_t smem = (size_t)n_warps * dk * sizeof(float);
    int st;
    if (dtype == TQ_F32)
        st = tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_attention_kernel<float>, grid, dim3(n_warps * 32), smem, stream,
                           (const float*)q, src, tok_pos, tok_seq, cu_seqlens, start_pos, scale, bias, n_dist, gate,
                           ldg, (float*)out, part, nh, nkv, dk, dv, n_splits);
    else if (dtype == TQ_BF16)
        st = tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_attention_kernel<bf16>, grid, dim3(n_warps * 32), smem, stream,
                           (const bf16*)q, src, tok_pos, tok_seq, cu_seqlens, start_pos, scale, bias, n_dist, gate, ldg,
                           (bf16*)out, part, nh, nkv, dk, dv, n_splits);
    else
        return (int)cudaErrorInvalidValue;
    if (st || n_splits == 1) return st;
    const dim3 mgrid(n_tokens, nh);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_attention_sum_kernel<float>, mgrid, dim3(64), 0, stream,
                             (const float*)part, gate, ldg, (float*)out, nh, dv, n_splits);
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_attention_sum_kernel<bf16>, mgrid, dim3(64), 0, stream,
                         (const float*)part, gate, ldg, (bf16*)out, nh, dv, n_splits);
}

// The sum of the splits alone (and the gate), for kernels that write the partial outputs themselves.
TQ_API int tq_sigmoid_attention_sum(const float* part, const float* gate, int ldg, void* out, int dtype, int n_tokens,
                                    int nh, int dv, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!part || n_splits < 1) return (int)cudaErrorInvalidValue;
    const dim3 mgrid(n_tokens, nh);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_attention_sum_kernel<float>, mgrid, dim3(64), 0, stream, part,
                             gate, ldg, (float*)out, nh, dv, n_splits);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, sigmoid_attention_sum_kernel<bf16>, mgrid, dim3(64), 0, stream, part,
                             gate, ldg, (bf16*)out, nh, dv, n_splits);
    return (int)cudaErrorInvalidValue;
}
