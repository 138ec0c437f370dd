// Mixers whose memory is a matrix per head that is carried from token to token: a d x e state S (d key
// channels, e value channels), float32, one per (sequence slot, head), updated once per token and read with a
// query.  Two update rules:
//
//   SCAN_DECAY   S_t = c_head * S_{t-1} + k_t v_t^T                       (a constant decay per head)
//   SCAN_DELTA   S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T
//                with u_t = k_t / sqrt(|k_t|^2 + unit_eps)                (the generalised delta rule: a decay per
//                key channel, and the removal of what the state holds along the unit key, at a rate per channel)
//   SCAN_GATED   S_t = g_t S_{t-1} + k_t (dt_t v_t)^T,  o_t = S_t^T q_t + skip_head * v_t
//                (one decay g and one step size dt per head and token; several heads may share q and k)
//   SCAN_GATED_DELTA   S' = g_t S_{t-1};  u = beta_t (v_t - S'^T k_t);  S_t = S' + k_t u^T
//                (the delta rule with one decay and one write strength per head and token: the state first
//                fades, then what it holds along k_t is replaced by v_t at the rate beta_t)
//   o_t = S_t^T q_t  in all.  The last two take their per-token scalars ready-made ([T, H, 4] floats: g, then
//   dt or beta), the value columns may be narrower or wider than the keys, and head h reads the q/k vectors of
//   head h / qk_div.
//
// Everything here is float32: the state, and all that enters the recurrence.  Three kernels:
//
// scan_prepare   once per (token, head), from the float32 results of the projections, in place:
//                  SCAN_DELTA  decay logit -> w = exp(-exp(-1/2) * sigmoid(logit)); removal logit -> -(a * u)
//                              with a = sigmoid(logit); u into a buffer of its own
//                  SCAN_DECAY  q, k, v -> silu (if asked)
// linear_scan    the columns of S (value channels) never mix, so the work is cut by column: a block owns some
//                columns of one head of one sequence and walks the sequence's tokens of this step in order, every
//                thread a tile of 8 keys x 4 columns of the state in registers (a token's vectors are then read
//                from shared memory once per 32 products, not once per product).  The tokens' vectors come through
//                shared memory a chunk at a time, two stages deep (cp.async), the outputs leave a chunk at a time.
//                The state is read from the slot's row before the first token and written back after the last: a
//                prompt, a portion of a prompt and a decoded token are the same kernel.
//                grid (sequence, head, column tile).
// linear_step    steps in which every sequence brings one token (decoding): the state is all the traffic, so a
//                warp owns 32 neighbouring columns and a slice of the keys (whole 128-byte rows of the state per
//                load), and the slices meet in shared memory.  It makes the token's vectors itself (what
//                scan_prepare does for the scan), so a decode step is one launch.
//                grid (sequence, head, column tile of 32).
#include "common.cuh"

#define SCAN_DECAY 0
#define SCAN_DELTA 1
#define SCAN_GATED 2
#define SCAN_GATED_DELTA 3
#define SCAN_THREADS 128      // of the one-token kernel

struct ScanArgs {
    const float* q;           // [T, ldp] query vectors, head h at columns h*d (the pointers are already offset)
    const float* k;           // keys, same layout
    const float* v;           // values, head h at columns h*e
    const float* au;          // SCAN_DELTA: minus removal rate times unit key (after scan_prepare)
    int ldp;                  // row stride of q, k, v, au (one projection buffer)
    const float* u;           // SCAN_DELTA: unit keys [T, ldu]
    int ldu;
    const float* w;           // SCAN_DELTA: decay per key channel [T, ldw] (after scan_prepare)
    int ldw;
    const float* head_decay;  // SCAN_DECAY: [H]
    float* state;             // [slots, H, d, e]
    const int* cu_seqlens;    // [B + 1] first token of each sequence in this step
    const int* slots;         // [B]
    float* out;               // [T, ldo], head h at columns h*e
    int ldo;
    int H, d, e;
    int chunk;                // tokens staged at a time
    int vec;                  // every vector starts on a 16-byte boundary and d, e are multiples of four
    int silu;                 // linear_step, SCAN_DECAY: q, k, v pass through silu (nothing was prepared)
    float unit_eps;           // linear_step, SCAN_DELTA: au and w hold the logits still (nothing was prepared)
    const float* scal;        // SCAN_GATED*: [T, H, 4] per token and head: decay, then step size or write strength
    const float* skip;        // SCAN_GATED: [H] or null, o += skip_head * v
    int qk_div;               // head h reads the q/k vectors of head h / qk_div
    size_t state_stride;      // floats from one slot's states to the next
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}

// ---------------------------------------------------------------------------
// scan_prepare: a warp per (token, head).
// ---------------------------------------------------------------------------
__global__ void scan_prepare_delta_kernel(const float* __restrict__ k, float* __restrict__ a_logit, int ldp,
                                          float* __restrict__ w_logit, int ldw, float* __restrict__ u, int ldu,
                                          int n_rows, int H, int d, float unit_eps) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch();
    if (row >= n_rows) return;
    const int t = row / H, h = row - t * H;
    const float* kr = k + (size_t)t * ldp + h * d;
    float* ar = a_logit + (size_t)t * ldp + h * d;
    float* wr = w_logit + (size_t)t * ldw + h * d;
    float* ur = u + (size_t)t * ldu + h * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(kr[i], kr[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss + unit_eps);
    for (int i = lane; i < d; i += 32) {
        const float uu = kr[i] * inv;
        ur[i] = uu;
        ar[i] = -(sigmoidf_(ar[i]) * uu);
        wr[i] = expf(-0.6065306597126334f * sigmoidf_(wr[i]));
    }
}

__global__ void silu_columns_kernel(float* __restrict__ x, int ld, int n, size_t total) {
    pdl_wait();
    pdl_launch();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        float* p = x + t * ld + (idx - t * n);
        *p = siluf_(*p);
    }
}

// ---------------------------------------------------------------------------
// linear_scan.  A thread owns a tile of the state: RK = 8 keys (two groups of four, interleaved over the KG
// lanes that share its columns, so that the lanes' 16-byte reads of a token's vectors touch every bank once)
// by RC neighbouring columns.  KG lanes together cover the DP = 8 * KG (padded) keys of their columns; a
// block of THREADS covers CT = THREADS / KG * RC columns.  A warp's time per token is its instruction count
// times the latency between dependent instructions (the tokens are a chain), so RC = 1 with many warps is the
// form for few sequences, and RC = 4, which reads a token's vectors once for four columns, the form for many.
// ---------------------------------------------------------------------------
template <int MODE, int KG, int THREADS, int RC>
__global__ void __launch_bounds__(THREADS) linear_scan_kernel(ScanArgs a) {
    constexpr int RK = 8;
    constexpr int DP = KG * RK;
    constexpr int CT = THREADS / KG * RC;
    constexpr int NV = MODE == SCAN_DELTA ? 5 : 2;
    constexpr int SC = MODE >= SCAN_GATED ? 4 : 0;          // a token's scalars, in front of a stage
    // tokens whose instructions the compiler may interleave (measured: the rules with one decay per head gain
    // up to 10 % from four, 2,048 tokens of 16 heads of 128 x 128: 716 -> 643 us)
    constexpr int TOKENS_AT_ONCE = MODE >= SCAN_GATED ? 4 : 2;
    extern __shared__ __align__(16) float sm[];
    const int b = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * CT;
    const int hq = head / a.qk_div;
    const int tid = threadIdx.x, kg = tid % KG, cg = tid / KG;
    const int colb = col0 + cg * RC;           // this thread's first column
    const int d = a.d, e = a.e, TC = a.chunk;
    const int stage_floats = TC * (SC + NV * DP + CT);
    float* so = sm + 2 * stage_floats;         // [TC][CT] outputs of a chunk
    // the padding (keys d .. DP-1, columns past e) stays zero: q, k, u and a*u of a key that does not exist
    for (int i = tid; i < 2 * stage_floats; i += THREADS) sm[i] = 0.f;

    pdl_wait();
    pdl_launch();
    const int t0 = a.cu_seqlens[b], t1 = a.cu_seqlens[b + 1];
    const int slot = a.slots[b];
    float* st = a.state + (size_t)slot * a.state_stride + (size_t)head * d * e;
    float2 S[RK / 2][RC];                      // S[r][c] = keys 2r and 2r + 1 of this thread, column c
#pragma unroll
    for (int r = 0; r < RK; ++r) {
        const int key = ((r >> 2) * KG + kg) * 4 + (r & 3);
#pragma unroll
        for (int c = 0; c < RC; ++c) {
            const float x = (key < d && colb + c < e) ? st[(size_t)key * e + colb + c] : 0.f;
            if (r & 1) S[r >> 1][c].y = x; else S[r >> 1][c].x = x;
        }
    }
    const float c_head = MODE == SCAN_DECAY ? a.head_decay[head] : 0.f;
    const float skip = (MODE == SCAN_GATED && a.skip) ? a.skip[head] : 0.f;
    __syncthreads();

    // stage s holds, token by token: q[DP] k[DP] (u[DP] au[DP] w[DP]) and after all of them v[TC][CT]
    auto stage_in = [&](int base, int s) {
        const int n = min(TC, t1 - base);
        float* dsc = sm + s * stage_floats;
        float* dst = dsc + TC * SC;
        float* dv = dst + TC * NV * DP;
        const int cols = min(CT, e - col0);
        if (SC) {
            if (a.vec) {
                for (int tt = tid; tt < n; tt += THREADS)
                    cp_async16(dsc + tt * 4, a.scal + ((size_t)(base + tt) * a.H + head) * 4);
            } else {
                for (int idx = tid; idx < n * 2; idx += THREADS)
                    dsc[(idx >> 1) * 4 + (idx & 1)] = a.scal[((size_t)(base + (idx >> 1)) * a.H + head) * 4 + (idx & 1)];
            }
        }
        if (a.vec) {
            const int d4 = d >> 2, c4 = cols >> 2;
            for (int idx = tid; idx < n * d4; idx += THREADS) {
                const int tt = idx / d4, i = (idx - tt * d4) * 4;
                const size_t t = (size_t)(base + tt);
                float* row = dst + tt * NV * DP + i;
                cp_async16(row, a.q + t * a.ldp + hq * d + i);
                cp_async16(row + DP, a.k + t * a.ldp + hq * d + i);
                if (MODE == SCAN_DELTA) {
                    cp_async16(row + 2 * DP, a.u + t * a.ldu + head * d + i);
                    cp_async16(row + 3 * DP, a.au + t * a.ldp + head * d + i);
                    cp_async16(row + 4 * DP, a.w + t * a.ldw + head * d + i);
                }
            }
            if (CT % 4 == 0) {                 // (a block of fewer than four columns takes its values one by one, below)
                for (int idx = tid; idx < n * c4; idx += THREADS) {
                    const int tt = idx / c4, c = (idx - tt * c4) * 4;
                    cp_async16(dv + tt * CT + c, a.v + (size_t)(base + tt) * a.ldp + head * e + col0 + c);
                }
            }
        } else {
            for (int idx = tid; idx < n * d; idx += THREADS) {
                const int tt = idx / d, i = idx - tt * d;
                const size_t t = (size_t)(base + tt);
                float* row = dst + tt * NV * DP + i;
                row[0] = a.q[t * a.ldp + hq * d + i];
                row[DP] = a.k[t * a.ldp + hq * d + i];
                if (MODE == SCAN_DELTA) {
                    row[2 * DP] = a.u[t * a.ldu + head * d + i];
                    row[3 * DP] = a.au[t * a.ldp + head * d + i];
                    row[4 * DP] = a.w[t * a.ldw + head * d + i];
                }
            }
        }
        if (!a.vec || CT % 4 != 0) {
            for (int idx = tid; idx < n * cols; idx += THREADS) {
                const int tt = idx / cols, c = idx - tt * cols;
                dv[tt * CT + c] = a.v[(size_t)(base + tt) * a.ldp + head * e + col0 + c];
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    if (t0 < t1) stage_in(t0, 0);
    int s = 0;
    for (int base = t0; base < t1; base += TC, s ^= 1) {
        const int n = min(TC, t1 - base);
        if (base + TC < t1) {
            stage_in(base + TC, s ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* ssc = sm + s * stage_floats;
        const float* src = ssc + TC * SC;
        const float* sv = src + TC * NV * DP;
#pragma unroll TOKENS_AT_ONCE
        for (int tt = 0; tt < n; ++tt) {
            // Two neighbouring keys of one column share a 64-bit register pair, and the products run two at a
            // time (fma.rn.f32x2: each half is the IEEE fused multiply-add of the scalar instruction).
            const float4* pq = reinterpret_cast<const float4*>(src + tt * NV * DP) + kg;
            float2 vv[RC];
            float xr[RC];
#pragma unroll
            for (int c = 0; c < RC; ++c) {
                const float x = sv[tt * CT + cg * RC + c];
                xr[c] = x;
                vv[c] = make_float2(x, x);
            }
            float2 kk[RK / 2], qq[RK / 2];
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const float4 k4 = pq[DP / 4 + g * KG], q4 = pq[g * KG];
                kk[2 * g] = make_float2(k4.x, k4.y); kk[2 * g + 1] = make_float2(k4.z, k4.w);
                qq[2 * g] = make_float2(q4.x, q4.y); qq[2 * g + 1] = make_float2(q4.z, q4.w);
            }
            float2 o2[RC];
#pragma unroll
            for (int c = 0; c < RC; ++c) o2[c] = make_float2(0.f, 0.f);
            if (MODE == SCAN_DELTA) {
                float2 uu[RK / 2], na[RK / 2], ww[RK / 2];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const float4 u4 = pq[2 * (DP / 4) + g * KG], a4 = pq[3 * (DP / 4) + g * KG],
                                 w4 = pq[4 * (DP / 4) + g * KG];
                    uu[2 * g] = make_float2(u4.x, u4.y); uu[2 * g + 1] = make_float2(u4.z, u4.w);
                    na[2 * g] = make_float2(a4.x, a4.y); na[2 * g + 1] = make_float2(a4.z, a4.w);
                    ww[2 * g] = make_float2(w4.x, w4.y); ww[2 * g + 1] = make_float2(w4.z, w4.w);
                }
                float dot[RC];
#pragma unroll
                for (int c = 0; c < RC; ++c) {
                    float2 acc = __fmul2_rn(uu[0], S[0][c]);
#pragma unroll
                    for (int r = 1; r < RK / 2; ++r) acc = __ffma2_rn(uu[r], S[r][c], acc);
                    dot[c] = acc.x + acc.y;
                }
#pragma unroll
                for (int off = KG / 2; off > 0; off >>= 1) {
#pragma unroll
                    for (int c = 0; c < RC; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], off);
                }
#pragma unroll
                for (int c = 0; c < RC; ++c) {
                    const float2 dd = make_float2(dot[c], dot[c]);
#pragma unroll
                    for (int r = 0; r < RK / 2; ++r) {
                        S[r][c] = __ffma2_rn(ww[r], S[r][c], __ffma2_rn(kk[r], vv[c], __fmul2_rn(na[r], dd)));
                        o2[c] = __ffma2_rn(qq[r], S[r][c], o2[c]);
                    }
                }
            } else if (MODE == SCAN_GATED_DELTA) {
                const float g = ssc[tt * 4], beta = ssc[tt * 4 + 1];
                const float2 gg = make_float2(g, g);
                float dot[RC];
#pragma unroll
                for (int c = 0; c < RC; ++c) {
                    float2 acc = __fmul2_rn(kk[0], S[0][c]);
#pragma unroll
                    for (int r = 1; r < RK / 2; ++r) acc = __ffma2_rn(kk[r], S[r][c], acc);
                    dot[c] = acc.x + acc.y;
                }
#pragma unroll
                for (int off = KG / 2; off > 0; off >>= 1) {
#pragma unroll
                    for (int c = 0; c < RC; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], off);
                }
#pragma unroll
                for (int c = 0; c < RC; ++c) {
                    const float u = beta * (xr[c] - g * dot[c]);       // what is written along k: the faded state's
                    const float2 uu = make_float2(u, u);               // reading is taken out, the value put in
#pragma unroll
                    for (int r = 0; r < RK / 2; ++r) {
                        S[r][c] = __ffma2_rn(gg, S[r][c], __fmul2_rn(kk[r], uu));
                        o2[c] = __ffma2_rn(qq[r], S[r][c], o2[c]);
                    }
                }
            } else {
                float2 cc = make_float2(c_head, c_head);
                if (MODE == SCAN_GATED) {
                    const float g = ssc[tt * 4], dt = ssc[tt * 4 + 1];
                    cc = make_float2(g, g);
#pragma unroll
                    for (int c = 0; c < RC; ++c) vv[c] = make_float2(dt * xr[c], dt * xr[c]);
                }
#pragma unroll
                for (int c = 0; c < RC; ++c) {
#pragma unroll
                    for (int r = 0; r < RK / 2; ++r) {
                        S[r][c] = __ffma2_rn(cc, S[r][c], __fmul2_rn(kk[r], vv[c]));
                        o2[c] = __ffma2_rn(qq[r], S[r][c], o2[c]);
                    }
                }
            }
            float o[RC];
#pragma unroll
            for (int c = 0; c < RC; ++c) o[c] = o2[c].x + o2[c].y;
            // the columns' sums over the KG lanes: lanes first trade columns until each holds one column's
            // partial sum, then the lanes that hold the same column meet
            if constexpr (RC == 4) {
                const bool odd = kg & 1, high = kg & 2;
                const float r0 = __shfl_xor_sync(0xffffffffu, odd ? o[0] : o[2], 1);
                const float r1 = __shfl_xor_sync(0xffffffffu, odd ? o[1] : o[3], 1);
                const float a0 = (odd ? o[2] : o[0]) + r0, a1 = (odd ? o[3] : o[1]) + r1;
                const float r2 = __shfl_xor_sync(0xffffffffu, high ? a0 : a1, 2);
                float sum = (high ? a1 : a0) + r2;            // column (odd ? 2 : 0) + (high ? 1 : 0)
#pragma unroll
                for (int off = 4; off < KG; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (MODE == SCAN_GATED) sum = fmaf(skip, odd ? (high ? xr[3] : xr[2]) : (high ? xr[1] : xr[0]), sum);
                if (kg < 4) so[tt * CT + cg * RC + (odd ? 2 : 0) + (high ? 1 : 0)] = sum;
            } else if constexpr (RC == 2) {
                const bool odd = kg & 1;
                float sum = (odd ? o[1] : o[0]) + __shfl_xor_sync(0xffffffffu, odd ? o[0] : o[1], 1);
#pragma unroll
                for (int off = 2; off < KG; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (MODE == SCAN_GATED) sum = fmaf(skip, odd ? xr[1] : xr[0], sum);
                if (kg < 2) so[tt * CT + cg * RC + (odd ? 1 : 0)] = sum;
            } else {
                float sum = o[0];
#pragma unroll
                for (int off = KG / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (MODE == SCAN_GATED) sum = fmaf(skip, xr[0], sum);
                if (kg == 0) so[tt * CT + cg] = sum;
            }
        }
        __syncthreads();                       // the chunk is consumed (its stage may be refilled), so[] is whole
        const int cols = min(CT, e - col0);
        for (int idx = tid; idx < n * cols; idx += THREADS) {
            const int tt = idx / cols, c = idx - tt * cols;
            a.out[(size_t)(base + tt) * a.ldo + head * e + col0 + c] = so[tt * CT + c];
        }
    }
#pragma unroll
    for (int r = 0; r < RK; ++r) {
        const int key = ((r >> 2) * KG + kg) * 4 + (r & 3);
#pragma unroll
        for (int c = 0; c < RC; ++c)
            if (key < d && colb + c < e) st[(size_t)key * e + colb + c] = (r & 1) ? S[r >> 1][c].y : S[r >> 1][c].x;
    }
}

#define SCAN_SMEM_LIMIT (64 * 1024)
#define SCAN_SMEM_ALONE (116 * 1024)      // two such blocks do not fit the 228 KB of an SM

template <int MODE, int KG, int THREADS, int RC>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    constexpr int CT = THREADS / KG * RC, DP = KG * 8, NV = MODE == SCAN_DELTA ? 5 : 2, SC = MODE >= SCAN_GATED ? 4 : 0;
    ScanArgs args = a;
    const int per_token = 2 * (SC + NV * DP + CT) + CT;  // two stages and the outputs
    int chunk = 8;
    while (chunk > 1 && (size_t)chunk * per_token * sizeof(float) > SCAN_SMEM_LIMIT) chunk >>= 1;
    args.chunk = chunk;
    size_t smem = (size_t)chunk * per_token * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_scan_kernel<MODE, KG, THREADS, RC>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM_ALONE);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const dim3 grid(n_seqs, a.H, (a.e + CT - 1) / CT);
    // Fewer blocks than SMs: every block should have an SM to itself, since a block's pace is set by the SM's
    // shared-memory pipe.  The block scheduler does not see to that by itself (blocks that start while the
    // kernel before drains gather on the SMs that fall free first: measured, the same launch took 0.2 or 0.5 ms),
    // so such a block asks for more shared memory than half an SM has.
    if ((long long)grid.x * grid.y * grid.z <= tq_sm_count() && smem < SCAN_SMEM_ALONE) smem = SCAN_SMEM_ALONE;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, linear_scan_kernel<MODE, KG, THREADS, RC>, grid, dim3(THREADS), smem, stream,
                         args);
}

// Which form.  One column a thread while such blocks still find an SM each (a block that shares its SM's
// shared-memory pipe with another runs at half the pace), in blocks as large as still leave a block for a quarter
// of the SMs; four columns a thread beyond that.
template <int MODE, int KG>
static int pick_form(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    const long long sms = tq_sm_count();
    auto blocks = [&](int threads, int rc) {
        const int ct = threads / KG * rc;
        return (long long)n_seqs * a.H * ((a.e + ct - 1) / ct);
    };
    if (a.e >= 256 / KG * 4 && blocks(256, 1) > sms) return launch_scan<MODE, KG, 256, 4>(a, n_seqs, stream);
    if (a.e >= 256 / KG && blocks(256, 1) >= sms / 4) return launch_scan<MODE, KG, 256, 1>(a, n_seqs, stream);
    if (a.e >= 128 / KG && blocks(128, 1) >= sms / 4) return launch_scan<MODE, KG, 128, 1>(a, n_seqs, stream);
    if (KG < 32 || a.e >= 2) return launch_scan<MODE, KG, 64, 1>(a, n_seqs, stream);
    return launch_scan<MODE, KG, 32, 1>(a, n_seqs, stream);
}

template <int MODE>
static int dispatch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    if (a.d <= 32) return pick_form<MODE, 4>(a, n_seqs, stream);
    if (a.d <= 64) return pick_form<MODE, 8>(a, n_seqs, stream);
    if (a.d <= 128) return pick_form<MODE, 16>(a, n_seqs, stream);
    return pick_form<MODE, 32>(a, n_seqs, stream);
}

// ---------------------------------------------------------------------------
// linear_step: one token per sequence.  Warp w of a block owns keys w, w + 4, ... and 32 columns; partial dot
// products meet in shared memory.  The token's vectors are staged once per block.
// ---------------------------------------------------------------------------
template <int MODE, int KPW>      // KPW: keys per warp (d <= 4 * KPW)
__global__ void __launch_bounds__(SCAN_THREADS) linear_step_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int b = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int d = a.d, e = a.e, col = col0 + lane;
    const int hq = head / a.qk_div;
    const bool col_ok = col < e;
    float* sq = sm;                 // [d] each: q k (u au w)
    float* sk = sq + d;
    float* su = sk + d;
    float* sau = su + d;
    float* sw = sau + d;
    float* red = sm + (MODE == SCAN_DELTA ? 5 : 2) * d;       // [4] + pad, then [2][4][32]
    pdl_wait();
    pdl_launch();
    const int t = a.cu_seqlens[b];
    const int slot = a.slots[b];
    float* st = a.state + (size_t)slot * a.state_stride + (size_t)head * d * e;
    float S[KPW];
#pragma unroll
    for (int i = 0; i < KPW; ++i) {
        const int key = i * 4 + warp;
        S[i] = (col_ok && key < d) ? st[(size_t)key * e + col] : 0.f;
    }
    // the token's vectors, made here from the projections' results (one token: no prepare kernel runs before)
    float ss = 0.f;
    for (int i = tid; i < d; i += SCAN_THREADS) {
        float qv = a.q[(size_t)t * a.ldp + hq * d + i], kv = a.k[(size_t)t * a.ldp + hq * d + i];
        if (MODE == SCAN_DECAY && a.silu) { qv = siluf_(qv); kv = siluf_(kv); }
        sq[i] = qv;
        sk[i] = kv;
        if (MODE == SCAN_DELTA) {
            ss = fmaf(kv, kv, ss);
            sau[i] = sigmoidf_(a.au[(size_t)t * a.ldp + head * d + i]);
            sw[i] = expf(-0.6065306597126334f * sigmoidf_(a.w[(size_t)t * a.ldw + head * d + i]));
        }
    }
    float vj = col_ok ? a.v[(size_t)t * a.ldp + head * e + col] : 0.f;
    if (MODE == SCAN_DECAY && a.silu) vj = siluf_(vj);
    if (MODE == SCAN_DELTA) {
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        const float inv = 1.f / sqrtf((red[0] + red[1]) + (red[2] + red[3]) + a.unit_eps);
        for (int i = tid; i < d; i += SCAN_THREADS) {       // (each thread rewrites the entries it wrote)
            const float uu = sk[i] * inv;
            su[i] = uu;
            sau[i] = -(sau[i] * uu);
        }
    }
    __syncthreads();
    float dot = 0.f;
    float g = 0.f, s2 = 0.f;            // SCAN_GATED*: the token's decay, and its step size or write strength
    if (MODE >= SCAN_GATED) {
        g = a.scal[((size_t)t * a.H + head) * 4];
        s2 = a.scal[((size_t)t * a.H + head) * 4 + 1];
    }
    if (MODE == SCAN_DELTA || MODE == SCAN_GATED_DELTA) {
        const float* sd = MODE == SCAN_DELTA ? su : sk;
#pragma unroll
        for (int i = 0; i < KPW; ++i) {
            const int key = i * 4 + warp;
            if (key < d) dot = fmaf(sd[key], S[i], dot);
        }
        red[128 + warp * 32 + lane] = dot;
        __syncthreads();
        dot = (red[128 + lane] + red[160 + lane]) + (red[192 + lane] + red[224 + lane]);
    }
    float o = 0.f;
    const float c_head = MODE == SCAN_DECAY ? a.head_decay[head] : g;
    float vw = vj;                      // what is written along the key
    if (MODE == SCAN_GATED) vw = s2 * vj;
    if (MODE == SCAN_GATED_DELTA) vw = s2 * (vj - g * dot);
#pragma unroll
    for (int i = 0; i < KPW; ++i) {
        const int key = i * 4 + warp;
        if (key < d) {
            if (MODE == SCAN_DELTA) S[i] = fmaf(sw[key], S[i], fmaf(sk[key], vj, sau[key] * dot));
            else S[i] = fmaf(c_head, S[i], sk[key] * vw);
            o = fmaf(sq[key], S[i], o);
            if (col_ok) st[(size_t)key * e + col] = S[i];
        }
    }
    red[256 + warp * 32 + lane] = o;
    __syncthreads();
    if (warp == 0 && col_ok) {
        float sum = (red[256 + lane] + red[288 + lane]) + (red[320 + lane] + red[352 + lane]);
        if (MODE == SCAN_GATED && a.skip) sum = fmaf(a.skip[head], vj, sum);
        a.out[(size_t)t * a.ldo + head * e + col] = sum;
    }
}

template <int MODE>
static int dispatch_step(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    const dim3 grid(n_seqs, a.H, (a.e + 31) / 32);
    const size_t smem = ((MODE == SCAN_DELTA ? 5 : 2) * (size_t)a.d + 384) * sizeof(float);
#define TQ_STEP(K) return tq_launch_pdl(TQ_PDL_ELEMENTWISE, linear_step_kernel<MODE, K>, grid, dim3(SCAN_THREADS), smem, stream, a)
    if (a.d <= 32) TQ_STEP(8);
    if (a.d <= 64) TQ_STEP(16);
    if (a.d <= 128) TQ_STEP(32);
    TQ_STEP(64);
#undef TQ_STEP
}

// mode 0 (constant decay per head, head_decay [H]; with `silu` q, k, v first pass through silu, in place) or 1 (the
// generalised delta rule: w_logit [T, ldw] and the removal logits at a_logit become w and a * u in place, u is
// scratch [T, ldu]; e == d).  q, k, v, a_logit point into one float32 buffer of row stride ldp.  `single` says that
// every sequence brings exactly one token: one kernel then does everything and the buffers are left as they were.
// Key widths up to 256.
TQ_API int tq_linear_scan(int mode, float* q, float* k, float* v, float* a_logit, int ldp, float* w_logit, int ldw,
                          float* u, int ldu, const float* head_decay, int silu, float unit_eps, float* state,
                          const int* cu_seqlens, const int* slots, int n_seqs, int n_tokens, int single, float* out,
                          int ldo, int H, int d, int e, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (!q || !k || !v || !state || !cu_seqlens || !slots || !out || H <= 0 || H > 65535 || d <= 0 || d > 256 || e <= 0)
        return (int)cudaErrorInvalidValue;
    ScanArgs a{q, k, v, a_logit, ldp, u, ldu, w_logit, ldw, head_decay, state, cu_seqlens, slots, out, ldo, H, d, e, 0, 0,
               silu, unit_eps, nullptr, nullptr, 1, (size_t)H * d * e};
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    a.vec = (d % 4 == 0 && e % 4 == 0 && ldp % 4 == 0 && al(q) && al(k) && al(v)) ? 1 : 0;
    if (mode == SCAN_DECAY) {
        if (!head_decay) return (int)cudaErrorInvalidValue;
        if (single) return dispatch_step<SCAN_DECAY>(a, n_seqs, stream);
        if (silu) {
            const int threads = 256;
            for (int part = 0; part < 3; ++part) {
                float* x = part == 0 ? q : (part == 1 ? k : v);
                const int n = part == 2 ? H * e : H * d;
                const size_t total = (size_t)n_tokens * n;
                size_t blocks = (total + threads - 1) / threads;
                if (blocks > (size_t)tq_sm_count() * 16) blocks = (size_t)tq_sm_count() * 16;
                int st = tq_launch_pdl(TQ_PDL_ELEMENTWISE, silu_columns_kernel, dim3((int)blocks), dim3(threads), 0, stream,
                                       x, ldp, n, total);
                if (st) return st;
            }
        }
        return dispatch_scan<SCAN_DECAY>(a, n_seqs, stream);
    }
    if (mode == SCAN_DELTA) {
        if (!w_logit || !a_logit || e != d) return (int)cudaErrorInvalidValue;
        if (single) return dispatch_step<SCAN_DELTA>(a, n_seqs, stream);
        if (!u) return (int)cudaErrorInvalidValue;
        a.vec = a.vec && ldu % 4 == 0 && ldw % 4 == 0 && al(u) && al(w_logit) && al(a_logit);
        const int rows = n_tokens * H;
        int st = tq_launch_pdl(TQ_PDL_ELEMENTWISE, scan_prepare_delta_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream,
                               (const float*)k, a_logit, ldp, w_logit, ldw, u, ldu, rows, H, d, unit_eps);
        if (st) return st;
        return dispatch_scan<SCAN_DELTA>(a, n_seqs, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// The rules with one decay per head and token.  q, k [T, ldp] with H / qk_div heads of d, v [T, ldp] with H heads of
// e, all in one float32 buffer and ready (activations, unit lengths and scales applied); scal [T, H, 4] holds each
// token's decay and, with `delta`, its write strength beta (S' = g S; S = S' + k (beta (v - S'^T k))^T), else its
// step size dt (S = g S + k (dt v)^T, o += skip_head * v if skip is given).  state points at the first slot's
// [H, d, e] block; state_stride floats lie between slots.  `single`: one token per sequence.
TQ_API int tq_gated_scan(int delta, const float* q, const float* k, const float* v, int ldp, const float* scal,
                         const float* skip, int qk_div, float* state, long long state_stride, const int* cu_seqlens,
                         const int* slots, int n_seqs, int n_tokens, int single, float* out, int ldo, int H, int d,
                         int e, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (!q || !k || !v || !scal || !state || !cu_seqlens || !slots || !out || H <= 0 || H > 65535 || d <= 0 || d > 256 ||
        e <= 0 || qk_div <= 0 || H % qk_div || state_stride < (long long)H * d * e)
        return (int)cudaErrorInvalidValue;
    ScanArgs a{q, k, v, nullptr, ldp, nullptr, 0, nullptr, 0, nullptr, state, cu_seqlens, slots, out, ldo, H, d, e, 0, 0,
               0, 0.f, scal, skip, qk_div, (size_t)state_stride};
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    a.vec = (d % 4 == 0 && e % 4 == 0 && ldp % 4 == 0 && al(q) && al(k) && al(v) && al(scal)) ? 1 : 0;
    if (delta) {
        if (single) return dispatch_step<SCAN_GATED_DELTA>(a, n_seqs, stream);
        return dispatch_scan<SCAN_GATED_DELTA>(a, n_seqs, stream);
    }
    if (single) return dispatch_step<SCAN_GATED>(a, n_seqs, stream);
    return dispatch_scan<SCAN_GATED>(a, n_seqs, stream);
}
