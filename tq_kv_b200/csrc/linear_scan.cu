// Mixers whose memory is a matrix per head that is carried from token to token: a d x e state S (d key
// channels, e value channels), float32, one per (sequence slot, head), updated once per token and read with a
// query.  Two update rules share one kernel:
//
//   SCAN_DECAY   S_t = c_head * S_{t-1} + k_t v_t^T                       (a constant decay per head)
//   SCAN_DELTA   S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T
//                with u_t = k_t / sqrt(|k_t|^2 + unit_eps)                (the generalised delta rule: a decay per
//                key channel, and the removal of what the state holds along the unit key, at a rate per channel)
//   o_t = S_t^T q_t  in both.
//
// The columns of S (value channels) never mix, so the work is cut by column: a thread group of KS lanes owns one
// column, each lane DPL of its d entries in registers; a block owns CT = 128 / KS columns of one head of one
// sequence and walks the sequence's tokens of this step in order.  The per-token vectors are staged through
// shared memory a chunk of tokens at a time, and everything that enters the recurrence is made there in float32
// from the float32 results of the projections:
//   SCAN_DECAY   q, k, v pass through silu (ACT_SILU) or unchanged
//   SCAN_DELTA   w = exp(-exp(-1/2) * sigmoid(decay logit)), a = sigmoid(removal logit), u from k
// The state is read from the slot's row at the start and written back at the end: a prompt, a portion of a prompt
// and a single decoded token are the same kernel.  grid (sequence, head, column tile).
#include "common.cuh"

#define SCAN_DECAY 0
#define SCAN_DELTA 1
#define SCAN_THREADS 128

struct ScanArgs {
    const float* proj;        // [T, ld] float32 projections of the step's tokens
    int ld;
    int off_q, off_k, off_v;  // first column of the query / key / value vectors (heads side by side)
    int off_a;                // SCAN_DELTA: first column of the removal logits
    const float* decay_logit; // SCAN_DELTA: [T, ld_w] logits of the decay, heads side by side
    int ld_w;
    const float* head_decay;  // SCAN_DECAY: [H]
    float* state;             // [slots, H, d, e]
    const int* cu_seqlens;    // [B + 1] first token of each sequence in this step
    const int* slots;         // [B]
    float* out;               // [T, ldo], head h at columns h*e ..
    int ldo;
    int H, d, e;
    int silu;                 // SCAN_DECAY: q, k, v pass through silu
    float unit_eps;
    int chunk;                // tokens staged at a time
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.f + expf(-z)); }

template <int MODE, int DPL, int KS>
__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(ScanArgs a) {
    constexpr int CT = SCAN_THREADS / KS;
    extern __shared__ float sm[];
    const int b = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * CT;
    const int tid = threadIdx.x, ks = tid % KS, cl = tid / KS;
    const int col = col0 + cl;
    const int d = a.d, e = a.e, TC = a.chunk;
    const bool col_ok = col < e;
    // shared: q[TC][d] k[TC][d] (delta: u[TC][d] au[TC][d] w[TC][d]) v[TC][CT] o[TC][CT] inv[TC]
    float* sq = sm;
    float* sk = sq + TC * d;
    float* su = sk + TC * d;
    float* sau = MODE == SCAN_DELTA ? su + TC * d : su;
    float* sw = MODE == SCAN_DELTA ? sau + TC * d : su;
    float* sv = MODE == SCAN_DELTA ? sw + TC * d : su;
    float* so = sv + TC * CT;
    float* sinv = so + TC * CT;

    pdl_wait();
    pdl_launch();
    const int t0 = a.cu_seqlens[b], t1 = a.cu_seqlens[b + 1];
    const int slot = a.slots[b];
    float* st = a.state + ((size_t)slot * a.H + head) * (size_t)d * e;
    float S[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int key = ks * DPL + i;
        S[i] = (col_ok && key < d) ? st[(size_t)key * e + col] : 0.f;
    }
    const float c_head = MODE == SCAN_DECAY ? a.head_decay[head] : 0.f;

    for (int base = t0; base < t1; base += TC) {
        const int n = min(TC, t1 - base);
        __syncthreads();                                   // the chunk before has been consumed
        for (int idx = tid; idx < n * d; idx += SCAN_THREADS) {
            const int tt = idx / d, i = idx - tt * d;
            const float* row = a.proj + (size_t)(base + tt) * a.ld + head * d + i;
            float q = row[a.off_q], k = row[a.off_k];
            if (MODE == SCAN_DECAY && a.silu) { q = siluf_(q); k = siluf_(k); }
            sq[idx] = q;
            sk[idx] = k;
            if (MODE == SCAN_DELTA) {
                const float lw = a.decay_logit[(size_t)(base + tt) * a.ld_w + head * d + i];
                sw[idx] = expf(-0.6065306597126334f * sigmoidf_(lw));
                sau[idx] = sigmoidf_(row[a.off_a]);        // the removal rate; times u below
            }
        }
        for (int idx = tid; idx < n * CT; idx += SCAN_THREADS) {
            const int tt = idx / CT, c = idx - tt * CT;
            float v = 0.f;
            if (col0 + c < e) {
                v = a.proj[(size_t)(base + tt) * a.ld + a.off_v + head * e + col0 + c];
                if (MODE == SCAN_DECAY && a.silu) v = siluf_(v);
            }
            sv[idx] = v;
        }
        __syncthreads();
        if (MODE == SCAN_DELTA) {
            // unit keys: a warp per token sums k^2
            for (int tt = tid >> 5; tt < n; tt += SCAN_THREADS >> 5) {
                float ss = 0.f;
                for (int i = tid & 31; i < d; i += 32) ss = fmaf(sk[tt * d + i], sk[tt * d + i], ss);
                ss = warp_sum(ss);
                if ((tid & 31) == 0) sinv[tt] = 1.f / sqrtf(ss + a.unit_eps);
            }
            __syncthreads();
            for (int idx = tid; idx < n * d; idx += SCAN_THREADS) {
                const float u = sk[idx] * sinv[idx / d];
                su[idx] = u;
                sau[idx] *= u;
            }
            __syncthreads();
        }
        for (int tt = 0; tt < n; ++tt) {
            const float* pq = sq + tt * d + ks * DPL;
            const float* pk = sk + tt * d + ks * DPL;
            const float vj = sv[tt * CT + cl];
            float o = 0.f;
            if (MODE == SCAN_DELTA) {
                const float* pu = su + tt * d + ks * DPL;
                const float* pau = sau + tt * d + ks * DPL;
                const float* pw = sw + tt * d + ks * DPL;
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < DPL; ++i)
                    if (ks * DPL + i < d) dot = fmaf(pu[i], S[i], dot);
#pragma unroll
                for (int off = KS / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
#pragma unroll
                for (int i = 0; i < DPL; ++i)
                    if (ks * DPL + i < d) {
                        S[i] = fmaf(pw[i], S[i], fmaf(pk[i], vj, -pau[i] * dot));
                        o = fmaf(pq[i], S[i], o);
                    }
            } else {
#pragma unroll
                for (int i = 0; i < DPL; ++i)
                    if (ks * DPL + i < d) {
                        S[i] = fmaf(c_head, S[i], pk[i] * vj);
                        o = fmaf(pq[i], S[i], o);
                    }
            }
#pragma unroll
            for (int off = KS / 2; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (ks == 0) so[tt * CT + cl] = o;
        }
        __syncthreads();
        for (int idx = tid; idx < n * CT; idx += SCAN_THREADS) {
            const int tt = idx / CT, c = idx - tt * CT;
            if (col0 + c < e) a.out[(size_t)(base + tt) * a.ldo + head * e + col0 + c] = so[idx];
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int key = ks * DPL + i;
            if (key < d) st[(size_t)key * e + col] = S[i];
        }
    }
}

template <int MODE, int DPL, int KS>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    constexpr int CT = SCAN_THREADS / KS;
    ScanArgs args = a;
    const int per_token = (MODE == SCAN_DELTA ? 5 : 2) * a.d + 2 * CT + 1;
    int chunk = 16;
    while (chunk > 1 && (size_t)chunk * per_token * sizeof(float) > 40 * 1024) chunk >>= 1;
    args.chunk = chunk;
    const size_t smem = (size_t)chunk * per_token * sizeof(float);
    const dim3 grid(n_seqs, a.H, (a.e + CT - 1) / CT);
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, linear_scan_kernel<MODE, DPL, KS>, grid, dim3(SCAN_THREADS), smem, stream,
                         args);
}

template <int MODE>
static int dispatch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    if (a.d <= 32) return launch_scan<MODE, 8, 4>(a, n_seqs, stream);
    if (a.d <= 64) return launch_scan<MODE, 16, 4>(a, n_seqs, stream);
    if (a.d <= 128) return launch_scan<MODE, 16, 8>(a, n_seqs, stream);
    return launch_scan<MODE, 32, 8>(a, n_seqs, stream);
}

// mode 0: constant decay per head (head_decay [H]; `silu` applies silu to q, k, v); mode 1: the generalised delta
// rule (decay logits [T, ld_w], removal logits at column off_a of proj, e == d).  Key widths up to 256.
TQ_API int tq_linear_scan(int mode, const float* proj, int ld, int off_q, int off_k, int off_v, int off_a,
                          const float* decay_logit, int ld_w, const float* head_decay, int silu, float unit_eps,
                          float* state, const int* cu_seqlens, const int* slots, int n_seqs, float* out, int ldo,
                          int H, int d, int e, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!proj || !state || !cu_seqlens || !slots || !out || H <= 0 || H > 65535 || d <= 0 || d > 256 || e <= 0)
        return (int)cudaErrorInvalidValue;
    ScanArgs a{proj, ld, off_q, off_k, off_v, off_a, decay_logit, ld_w, head_decay, state, cu_seqlens, slots, out, ldo,
               H, d, e, silu, unit_eps, 0};
    if (mode == SCAN_DECAY) {
        if (!head_decay) return (int)cudaErrorInvalidValue;
        return dispatch_scan<SCAN_DECAY>(a, n_seqs, stream);
    }
    if (mode == SCAN_DELTA) {
        if (!decay_logit) return (int)cudaErrorInvalidValue;
        return dispatch_scan<SCAN_DELTA>(a, n_seqs, stream);
    }
    return (int)cudaErrorInvalidValue;
}
