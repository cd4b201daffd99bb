// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float32
// accumulate, online softmax in float32): one kernel for decode, one for prefill, one to merge splits.
//
// Decode (`attn_decode_kernel`): one CTA per (token, kv head, split of the key range), four warps.
// The query heads that share the kv head are the rows of the 16-row MMA tile, so keys and values are
// read once per group.  A decode step is a stream of the cache from HBM, so K and V go straight from
// global memory into MMA fragments with 16-byte loads and no shared-memory staging: the contraction
// index of Q.K^T (the head dimension) and the output columns of P.V may be permuted freely, and the
// permutations are chosen so that each thread's fragment elements are contiguous in memory.  Each
// warp keeps its own running maximum, sum and output; the warps are merged in shared memory, the
// splits by `attn_combine_kernel` in a fixed order.
//
// Prefill (`attn_prefill_kernel`): one CTA per (64-query tile of one sequence, query head), four
// warps of 16 query rows.  Key/value tiles of 64 positions (one cache page) are staged in swizzled
// shared memory with cp.async, double buffered, and read with ldmatrix.  Causal and window masks are
// applied in the tiles they cut; tiles outside the visible range are skipped.  Because keys and
// values come from the cache, a prompt that continues a cached prefix runs through the same kernel.
//
// Replaces the reference's per-head attn_qk / softmax / attn_v launches (pkg/gpu/cuda/ptx.go:679-889,
// host loop pkg/gpu/cuda/driver.c:411-465).
#include "tma_util.cuh"

namespace {

constexpr int PAGE = 64;

__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Pairs of float32 in one 64-bit register for the packed arithmetic of sm_100 (two results per issue slot).
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ void st_dsmem_f32(uint32_t local_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

__device__ __forceinline__ float ld_dsmem_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// ------------------------------------------------------------------------------------------- decode
// Rows of the MMA tile: query head r of the group (r < G <= 16).  Fragment conventions (g = lane / 4,
// t = lane % 4): A regs {row g, row g+8} x {k low, k high}; B regs (k = 2t..2t+1 | 8+2t.., n = g);
// C regs c0,c1 = row g, cols 2t, 2t+1; c2,c3 = row g+8.
template <int D>
__global__ void __launch_bounds__(128) attn_decode_kernel(
    const bf16* q, const bf16* k_pool, const bf16* v_pool,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int nq, int nkv, float scale_log2, int window, int nsplit,
    const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    constexpr int NCH = D / 32;      // 32-wide chunks of the head dimension for Q.K^T
    constexpr int NDB = D / 64;      // 64-wide blocks of output columns for P.V
    constexpr int NT = D / 8;        // output n-tiles
    __shared__ float sm_o[4][16][D];
    __shared__ float sm_ml[4][16][2];
    const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = nq / nkv;
    const int b = seq_of_token[tok];
    const int pos = b >= 0 ? positions[tok] : -1;

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (b >= 0) {
        int lo = 0;
        if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
        const int first = lo >> 4, last = pos >> 4;
        const int ntiles = last - first + 1;
        const int tps = (ntiles + nsplit - 1) / nsplit;
        const int t_begin = first + split * tps;
        const int t_end = min(last + 1, t_begin + tps);

        // Q fragments: row g (and g+8) of the group, permuted head dimension (see file header)
        uint32_t qa[NCH][2][4];
        {
            const bf16* q0 = q + ((size_t)tok * nq + (size_t)kvh * G) * D;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                uint4 w0 = make_uint4(0, 0, 0, 0), w1 = make_uint4(0, 0, 0, 0);
                if (g < G) w0 = ldg16(q0 + (size_t)g * D + c * 32 + t * 8);
                if (g + 8 < G) w1 = ldg16(q0 + (size_t)(g + 8) * D + c * 32 + t * 8);
                qa[c][0][0] = w0.x; qa[c][0][1] = w1.x; qa[c][0][2] = w0.y; qa[c][0][3] = w1.y;
                qa[c][1][0] = w0.z; qa[c][1][1] = w1.z; qa[c][1][2] = w0.w; qa[c][1][3] = w1.w;
            }
        }
        const int* pt = page_table + (size_t)b * max_pages;
        for (int kt = t_begin + warp; kt < t_end; kt += 4) {
            const int key0 = kt << 4;
            const int page = gg_page(pt, key0 / PAGE, max_pages, pb, 42);
            const size_t base = (((size_t)page * nkv + kvh) * PAGE + (key0 % PAGE)) * D;
            // ---- S = Q K^T for 16 keys (two n-tiles of 8)
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
                const bf16* kr = k_pool + base + (size_t)(j * 8 + g) * D + t * 8;
                uint4 kw[NCH];
#pragma unroll
                for (int c = 0; c < NCH; ++c) kw[c] = ldg16(kr + c * 32);
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    mma16816(s[j], qa[c][0], kw[c].x, kw[c].y);
                    mma16816(s[j], qa[c][1], kw[c].z, kw[c].w);
                }
            }
            // ---- V rows of this thread: keys 2t, 2t+1, 8+2t, 9+2t; columns db*64 + g*8 .. +8
            uint4 vw[NDB][4];
            {
                const bf16* vr = v_pool + base + g * 8;
#pragma unroll
                for (int db = 0; db < NDB; ++db) {
                    vw[db][0] = ldg16(vr + (size_t)(2 * t) * D + db * 64);
                    vw[db][1] = ldg16(vr + (size_t)(2 * t + 1) * D + db * 64);
                    vw[db][2] = ldg16(vr + (size_t)(8 + 2 * t) * D + db * 64);
                    vw[db][3] = ldg16(vr + (size_t)(9 + 2 * t) * D + db * 64);
                }
            }
            // ---- mask, online softmax (log2 domain)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kidx = key0 + j * 8 + 2 * t + (e & 1);
                    const float v = (kidx >= lo && kidx <= pos) ? s[j][e] * scale_log2 : -INFINITY;
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            uint32_t pa[4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float mn = fmaxf(m[r], mx[r]);
                const float mu = mn == -INFINITY ? 0.f : mn;
                const float corr = fast_exp2(m[r] - mu);
                m[r] = mn;
                const float p00 = fast_exp2(s[0][2 * r] - mu), p01 = fast_exp2(s[0][2 * r + 1] - mu);
                const float p10 = fast_exp2(s[1][2 * r] - mu), p11 = fast_exp2(s[1][2 * r + 1] - mu);
                l[r] = l[r] * corr + (p00 + p01 + p10 + p11);
                pa[r] = pack_bf16(p00, p01);          // A reg r: row g + 8r, keys 2t, 2t+1
                pa[2 + r] = pack_bf16(p10, p11);      // A reg 2+r: row g + 8r, keys 8+2t, 9+2t
#pragma unroll
                for (int i = 0; i < NT; ++i) { o[i][2 * r] *= corr; o[i][2 * r + 1] *= corr; }
            }
            // ---- O += P V
#pragma unroll
            for (int db = 0; db < NDB; ++db) {
                const uint32_t* a0 = reinterpret_cast<const uint32_t*>(&vw[db][0]);
                const uint32_t* a1 = reinterpret_cast<const uint32_t*>(&vw[db][1]);
                const uint32_t* a2 = reinterpret_cast<const uint32_t*>(&vw[db][2]);
                const uint32_t* a3 = reinterpret_cast<const uint32_t*>(&vw[db][3]);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    mma16816(o[db * 8 + 2 * w], pa, __byte_perm(a0[w], a1[w], 0x5410), __byte_perm(a2[w], a3[w], 0x5410));
                    mma16816(o[db * 8 + 2 * w + 1], pa, __byte_perm(a0[w], a1[w], 0x7632), __byte_perm(a2[w], a3[w], 0x7632));
                }
            }
        }
    }
    // ---- merge the four warps
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int db = i >> 3, jn = i & 7;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = g + 8 * (e >> 1);
            const int col = db * 64 + (2 * t + (e & 1)) * 8 + jn;    // undo the column permutation
            sm_o[warp][row][col] = o[i][e];
        }
    }
    if (t == 0) {
        sm_ml[warp][g][0] = m[0]; sm_ml[warp][g][1] = l[0];
        sm_ml[warp][g + 8][0] = m[1]; sm_ml[warp][g + 8][1] = l[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int r = idx / D, c = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[w][r][0]);
        float L = 0.f, acc = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = fast_exp2(sm_ml[w][r][0] - M);
                L += sm_ml[w][r][1] * f;
                acc += sm_o[w][r][c] * f;
            }
        }
        const int head = kvh * G + r;
        if (nsplit == 1) {
            out[((size_t)tok * nq + head) * D + c] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t pi = ((size_t)tok * nq + head) * nsplit + split;
            part_o[pi * D + c] = acc;
            if (c == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
}

template <int D>
__global__ void attn_combine_kernel(const float* part_o, const float* part_ml,
                                    bf16* __restrict__ out, int nsplit) {
    pdl_launch();
    pdl_wait();
    const size_t row = blockIdx.x;         // token * nq + head
    const int c = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(row * nsplit + s) * 2]);
    float L = 0.f, acc = 0.f;
    if (M != -INFINITY) {
        for (int s = 0; s < nsplit; ++s) {
            const float f = fast_exp2(part_ml[(row * nsplit + s) * 2] - M);
            L += part_ml[(row * nsplit + s) * 2 + 1] * f;
            acc += part_o[(row * nsplit + s) * D + c] * f;
        }
    }
    out[row * D + c] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

// ------------------------------------------------------------------------------------------- prefill
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

// element (row, 16-byte chunk) of a [rows][D] bf16 tile with the chunk index XOR-swizzled by the row
template <int D> __device__ __forceinline__ bf16* sw(bf16* tile, int row, int chunk) {
    return tile + row * D + ((chunk ^ (row & 7)) << 3);
}

template <int D>
__global__ void __launch_bounds__(128) attn_prefill_kernel(
    const bf16* q, const bf16* k_pool, const bf16* v_pool, bf16* __restrict__ out,
    const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int n_seqs, int nq, int nkv, float scale_log2, int window,
    const PageBounds pb) {
    pdl_wait();      // no early release of the next kernel: many waves of CTAs that exclude its CTAs from their SMs
    constexpr int CH = D / 8;        // 16-byte chunks per row
    constexpr int KS = D / 16;       // k-steps of Q.K^T
    constexpr int NT = D / 8;        // output n-tiles
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + 64 * D;          // two stages
    bf16* Vs = Ks + 2 * 64 * D;      // two stages

    // which (sequence, query tile) is this CTA?  tiles are numbered sequence by sequence
    int b = -1, tile = blockIdx.x, n_new = 0, tok0 = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const int a = cu_seqlens[i], e = cu_seqlens[i + 1];
        if (seq_of_token[a] < 0) continue;                 // padding row of a padded batch
        const int nt = (e - a + 63) >> 6;
        if (tile < nt) { b = i; n_new = e - a; tok0 = a; break; }
        tile -= nt;
    }
    if (b < 0) return;
    const int h = blockIdx.y, kvh = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = tile * 64;                              // first query row of this tile within the new tokens
    const int rows = min(64, n_new - row0);
    const int pos0 = ctx_lens[b] - n_new + row0;             // absolute position of query row 0
    const int* pt = page_table + (size_t)b * max_pages;

    int lo = 0;
    if (window > 0 && pos0 - window + 1 > 0) lo = pos0 - window + 1;
    const int kt_first = lo / PAGE, kt_last = (pos0 + rows - 1) / PAGE;

    // ---- stage Q (rows beyond the tile are zero) and the first K/V tile
    for (int idx = threadIdx.x; idx < 64 * CH; idx += 128) {
        const int r = idx / CH, c = idx - r * CH;
        bf16* dst = sw<D>(Qs, r, c);
        if (r < rows) cp_async16(dst, q + ((size_t)(tok0 + row0 + r) * nq + h) * D + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    auto load_kv = [&](int kt, int stage) {
        const size_t base = (((size_t)gg_page(pt, kt, max_pages, pb, 43) * nkv + kvh) * PAGE) * D;
        bf16* kd = Ks + stage * 64 * D;
        bf16* vd = Vs + stage * 64 * D;
        for (int idx = threadIdx.x; idx < 64 * CH; idx += 128) {
            const int r = idx / CH, c = idx - r * CH;
            cp_async16(sw<D>(kd, r, c), k_pool + base + (size_t)r * D + c * 8);
            cp_async16(sw<D>(vd, r, c), v_pool + base + (size_t)r * D + c * 8);
        }
    };
    load_kv(kt_first, 0);
    cp_async_commit();

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    uint32_t qa[KS][4];
    const int qrow = warp * 16;      // this warp's 16 query rows

    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        if (kt + 1 <= kt_last) load_kv(kt + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (kt == kt_first) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) ldsm_x4(qa[ks], sw<D>(Qs, qrow + (lane & 15), ks * 2 + (lane >> 4)));
        }
        const bf16* kd = Ks + stage * 64 * D;
        const bf16* vd = Vs + stage * 64 * D;
        // rows of this warp that can see any key of this tile?  (whole-warp decision, keeps barriers aligned)
        const int key0 = kt * PAGE;
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {       // pairs of n-tiles (16 keys)
                uint32_t kb[4];
                ldsm_x4(kb, sw<D>(const_cast<bf16*>(kd), np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                mma16816(s[2 * np], qa[ks], kb[0], kb[1]);
                mma16816(s[2 * np + 1], qa[ks], kb[2], kb[3]);
            }
        }
        // ---- mask + online softmax
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = qrow + g + 8 * (e >> 1);
                const int p = pos0 + r;
                const int kidx = key0 + nt * 8 + 2 * t + (e & 1);
                bool ok = kidx <= p;
                if (window > 0) ok = ok && (kidx > p - window);
                const float v = ok ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float mu[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(m[r], mx[r]);
            mu[r] = mn == -INFINITY ? 0.f : mn;
            const float corr = fast_exp2(m[r] - mu[r]);
            m[r] = mn;
            l[r] *= corr;
#pragma unroll
            for (int i = 0; i < NT; ++i) { o[i][2 * r] *= corr; o[i][2 * r + 1] *= corr; }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = fast_exp2(s[nt][e] - mu[e >> 1]);
                s[nt][e] = p;
                l[e >> 1] += p;
            }
        // ---- O += P V  (k = 16 keys per step, four steps per tile)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t vb[4];
                ldsm_x4_trans(vb, sw<D>(const_cast<bf16*>(vd), kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
                mma16816(o[2 * np], pa, vb[0], vb[1]);
                mma16816(o[2 * np + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();     // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();
    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = qrow + g + 8 * r;
        if (row >= rows) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        bf16* dst = out + ((size_t)(tok0 + row0 + row) * nq + h) * D;
#pragma unroll
        for (int i = 0; i < NT; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}


// ------------------------------------------------------------------------------------------- decode, TMA ring
// The same work as attn_decode_kernel with the cache streamed by TMA: one producer thread keeps a
// ring of whole pages (64 keys: K and V, [64 x 64]-column boxes, 128-byte swizzle) in flight, four
// consumer warps take 16 keys of each page, read fragments with ldmatrix and keep their own running
// maximum, sum and output; they are merged at the end as in the other kernel.  The copy engine
// decouples the loads from the arithmetic, which a warp that loads and computes in turn cannot.
// Largest cluster of splits: 8 is what every device takes; 16 needs the non-portable opt-in, which the
// launcher asks for once and falls back from (attn_max_cluster).
constexpr int MAX_ATT_CLUSTER = 16;

// What the other CTAs of a cluster push into this one (beyond the ring, so that they need not wait for it): their
// partial outputs for the slices of 32 this CTA merges, [rank][round][32], and their (max, sum) per query head.
constexpr int ATT_PUSH_MAX_OUT = 1024;                               // G * D up to which the splits are pushed
constexpr int ATT_RECV_O = (ATT_PUSH_MAX_OUT + 32 * 16) * 4;         // bytes: rank * rounds * 32 <= G * D + 32 * cs
constexpr int ATT_RECV_ML = 16 * 16 * 2 * 4;
constexpr int ATT_RECV_BYTES = ATT_RECV_O + ATT_RECV_ML;


template <int D, int STAGES>
__global__ void __launch_bounds__(160) attn_decode_tma_kernel(
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
    const bf16* q, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int nq, int nkv, float scale_log2, int window, int nsplit,
    int cluster_reduce, int early_release, int n_pages, int* __restrict__ status) {
    // A grid that is resident as a whole lets the next kernel's CTAs in at once: they share the SMs' free
    // shared memory and start fetching weights.  A grid of several waves releases only after its pages (the
    // rule on dependent launches in common.cuh): until then its own waiting CTAs should get the SMs.
    if (early_release) pdl_launch();
    constexpr int HALVES = D / 64;
    constexpr int BOX_BYTES = 64 * 64 * 2;                 // 8 KB
    constexpr int STAGE_BYTES = 2 * HALVES * BOX_BYTES;    // K halves then V halves
    constexpr int KS = D / 16, NT = D / 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    volatile int* abort_flag = (volatile int*)(empty + STAGES);
    float* recv_o = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);      // see ATT_RECV_BYTES
    float* recv_ml = recv_o + ATT_RECV_O / 4;

    const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = nq / nkv;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { tma::mbar_init(&full[s], 1); tma::mbar_init(&empty[s], 4); }
        *abort_flag = 0;
        tma::mbar_fence_init();
        tma::prefetch_map(&tmK);
        tma::prefetch_map(&tmV);
    }
    __syncthreads();
    // The step's integer inputs (positions, sequence rows, page tables) were copied to the device before the
    // step's first kernel started.  Of the cache, the kernels of this step write only position `pos` (one new
    // token per sequence), which lies in page pos / 64; every earlier page was written by earlier steps.  So
    // the producer starts streaming those pages while the projection before this kernel is still finishing,
    // and waits for it only before the page that holds the new token; the consumers wait before they read q.
    const int b = seq_of_token[tok];
    const int pos = b >= 0 ? positions[tok] : -1;

    int lo = 0, p_begin = 0, p_end = 0;
    if (b >= 0) {
        if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
        const int first = lo / PAGE, last = pos / PAGE;
        const int pps = (last - first + 1 + nsplit - 1) / nsplit;
        p_begin = first + split * pps;
        p_end = min(last + 1, p_begin + pps);
    }
    const int npg = max(0, p_end - p_begin);

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (warp == 4) {
        if (lane == 0) {
            const int* pt = page_table + (size_t)b * max_pages;
            const int newest = pos / PAGE;
            bool waited = false;
            for (int i = 0; i < npg; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                if (!waited && p_begin + i >= newest) { pdl_wait(); waited = true; }
                if (!tma::mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, 11)) break;
                tma::mbar_expect_tx(&full[s], STAGE_BYTES);
                const int row = (gg_page(pt, p_begin + i, max_pages, PageBounds{n_pages, status}, 44) * nkv + kvh) * PAGE;
                uint8_t* dst = smem + s * STAGE_BYTES;
#pragma unroll
                for (int hf = 0; hf < HALVES; ++hf) {
                    tma::load_2d(dst + hf * BOX_BYTES, &tmK, &full[s], hf * 64, row);
                    tma::load_2d(dst + (HALVES + hf) * BOX_BYTES, &tmV, &full[s], hf * 64, row);
                }
            }
        }
    } else if (npg > 0) {
        // Q fragments in the standard A layout: row = head of the group, k = head dimension
        uint32_t qa[KS][4];
        pdl_wait();
        {
            const bf16* q0 = q + ((size_t)tok * nq + (size_t)kvh * G) * D;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int c = ks * 16 + 2 * t;
                qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + c) : 0u;
                qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + c) : 0u;
                qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + c + 8) : 0u;
                qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + c + 8) : 0u;
            }
        }
        const int krow = warp * 16;     // this warp's 16 keys of every page
        for (int i = 0; i < npg; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
            if (!tma::mbar_wait(&full[s], ph, abort_flag, status, 12)) break;
            const uint8_t* st = smem + s * STAGE_BYTES;
            const int key0 = (p_begin + i) * PAGE + krow;
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = 0.f;
            sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
            if (key0 <= pos && key0 + 15 >= lo) {      // whole-warp decision: any visible key among these 16?
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const bf16* box = reinterpret_cast<const bf16*>(st + (ks >> 2) * BOX_BYTES);
                    uint32_t kb[4];
                    ldsm_x4(kb, sw<64>(const_cast<bf16*>(box), krow + (lane & 7) + ((lane >> 4) << 3), (ks & 3) * 2 + ((lane >> 3) & 1)));
                    mma16816(sc[0], qa[ks], kb[0], kb[1]);
                    mma16816(sc[1], qa[ks], kb[2], kb[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int kidx = key0 + j * 8 + 2 * t + (e & 1);
                        const float v = (kidx >= lo && kidx <= pos) ? sc[j][e] * scale_log2 : -INFINITY;
                        sc[j][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                uint32_t pa[4];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    const float mn = fmaxf(m[r], mx[r]);
                    const float mu = mn == -INFINITY ? 0.f : mn;
                    const float corr = fast_exp2(m[r] - mu);
                    m[r] = mn;
                    const float p00 = fast_exp2(sc[0][2 * r] - mu), p01 = fast_exp2(sc[0][2 * r + 1] - mu);
                    const float p10 = fast_exp2(sc[1][2 * r] - mu), p11 = fast_exp2(sc[1][2 * r + 1] - mu);
                    l[r] = l[r] * corr + (p00 + p01 + p10 + p11);
                    pa[r] = pack_bf16(p00, p01);
                    pa[2 + r] = pack_bf16(p10, p11);
#pragma unroll
                    for (int n = 0; n < NT; ++n) { o[n][2 * r] *= corr; o[n][2 * r + 1] *= corr; }
                }
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    const bf16* box = reinterpret_cast<const bf16*>(st + (HALVES + (np >> 2)) * BOX_BYTES);
                    uint32_t vb[4];
                    ldsm_x4_trans(vb, sw<64>(const_cast<bf16*>(box), krow + (lane & 7) + (((lane >> 3) & 1) << 3), (np & 3) * 2 + (lane >> 4)));
                    mma16816(o[2 * np], pa, vb[0], vb[1]);
                    mma16816(o[2 * np + 1], pa, vb[2], vb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&empty[s]);
        }
    }
    pdl_wait();               // (returns at once where it was already called) the output buffer is free from here
    if (!early_release) pdl_launch();
    __syncthreads();          // all pages consumed (or the CTA gave up): the ring can be reused for the merge
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }       // let copies in flight land before the CTA goes away
        __syncthreads();
    }
    float* sm_o = reinterpret_cast<float*>(smem);                 // [4][16][D]
    float* sm_ml = sm_o + 4 * 16 * D;                             // [4][16][2]
    float* res_o = sm_ml + 4 * 16 * 2;                            // [16][D]  this CTA's merged output (cluster form)
    float* res_ml = res_o + 16 * D;                               // [16][2]
    if (warp < 4) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        }
        // only the G rows that are query heads go on (the MMA tile has 16)
        if (g < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n)
                *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g) * D + n * 8 + 2 * t]) = make_float2(o[n][0], o[n][1]);
            if (t == 0) { sm_ml[(warp * 16 + g) * 2] = m[0]; sm_ml[(warp * 16 + g) * 2 + 1] = l[0]; }
        }
        if (g + 8 < G) {
#pragma unroll
            for (int n = 0; n < NT; ++n)
                *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g + 8) * D + n * 8 + 2 * t]) = make_float2(o[n][2], o[n][3]);
            if (t == 0) { sm_ml[(warp * 16 + g + 8) * 2] = m[1]; sm_ml[(warp * 16 + g + 8) * 2 + 1] = l[1]; }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int r = idx / D, c = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = fast_exp2(sm_ml[(w * 16 + r) * 2] - M);
                L += sm_ml[(w * 16 + r) * 2 + 1] * f;
                acc += sm_o[(w * 16 + r) * D + c] * f;
            }
        }
        const int head = kvh * G + r;
        if (nsplit == 1) {
            out[((size_t)tok * nq + head) * D + c] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else if (cluster_reduce && G * D <= ATT_PUSH_MAX_OUT) {
            // straight into the shared memory of the CTA that merges this output (slices of 32 go round the
            // ranks), and this head's (max, sum) to every CTA: no load has to cross the cluster afterwards
            const int chunk = idx >> 5, owner = chunk % nsplit, round = chunk / nsplit;
            const int rounds = ((G * D + 31) / 32 + nsplit - 1) / nsplit;
            st_dsmem_f32(tma::smem_u32(recv_o + (split * rounds + round) * 32 + (idx & 31)), (uint32_t)owner, acc);
            if (c == 0) {
                for (int k = 0; k < nsplit; ++k) {
                    st_dsmem_f32(tma::smem_u32(recv_ml + (split * 16 + r) * 2), (uint32_t)k, M);
                    st_dsmem_f32(tma::smem_u32(recv_ml + (split * 16 + r) * 2 + 1), (uint32_t)k, L);
                }
            }
        } else if (cluster_reduce) {
            res_o[r * D + c] = acc;
            if (c == 0) { res_ml[r * 2] = M; res_ml[r * 2 + 1] = L; }
        } else {
            const size_t pi = ((size_t)tok * nq + head) * nsplit + split;
            part_o[pi * D + c] = acc;
            if (c == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
    if (cluster_reduce && G * D <= ATT_PUSH_MAX_OUT) {
        // The splits of one (token, kv head) form a cluster; what the ranks pushed is complete after one barrier,
        // and every CTA merges its slice of the G x D outputs, in rank order, from its own shared memory.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int rounds = ((G * D + 31) / 32 + nsplit - 1) / nsplit;
        for (int round = warp; round < rounds; round += 5) {
            const int idx = (round * nsplit + split) * 32 + lane;
            if (idx >= G * D) continue;
            const int r = idx / D;
            float M = -INFINITY;
            for (int k = 0; k < nsplit; ++k) M = fmaxf(M, recv_ml[(k * 16 + r) * 2]);
            float L = 0.f, acc = 0.f;
            if (M != -INFINITY) {
                for (int k = 0; k < nsplit; ++k) {
                    const float f = fast_exp2(recv_ml[(k * 16 + r) * 2] - M);
                    L += recv_ml[(k * 16 + r) * 2 + 1] * f;
                    acc += recv_o[(k * rounds + round) * 32 + lane] * f;
                }
            }
            out[((size_t)tok * nq + kvh * G) * D + idx] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        }
    } else if (cluster_reduce) {
        // (more than 1,024 outputs per kv head do not fit the receive area: the owner pulls instead)
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const uint32_t ro = tma::smem_u32(res_o), rm = tma::smem_u32(res_ml);
        for (int idx = split * blockDim.x + threadIdx.x; idx < G * D; idx += nsplit * blockDim.x) {
            const int r = idx / D, c = idx - r * D;
            float ms[MAX_ATT_CLUSTER], ls[MAX_ATT_CLUSTER], as[MAX_ATT_CLUSTER];
            float M = -INFINITY;
#pragma unroll
            for (int k = 0; k < MAX_ATT_CLUSTER; ++k) {
                if (k < nsplit) {
                    ms[k] = ld_dsmem_f32(rm + 4u * (r * 2), k);
                    ls[k] = ld_dsmem_f32(rm + 4u * (r * 2 + 1), k);
                    as[k] = ld_dsmem_f32(ro + 4u * idx, k);
                } else { ms[k] = -INFINITY; ls[k] = 0.f; as[k] = 0.f; }
                M = fmaxf(M, ms[k]);
            }
            float L = 0.f, acc = 0.f;
            if (M != -INFINITY) {
#pragma unroll
                for (int k = 0; k < MAX_ATT_CLUSTER; ++k) {
                    const float f = fast_exp2(ms[k] - M);
                    L += ls[k] * f;
                    acc += as[k] * f;
                }
            }
            out[((size_t)tok * nq + kvh * G + r) * D + c] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
}

template <int D, int STAGES>
constexpr int decode_tma_smem() {
    constexpr int ring = STAGES * 4 * (D / 64) * 64 * 64;     // bytes: STAGES * 2 * HALVES * 8 KB
    constexpr int merge = (5 * 16 * D + 5 * 16 * 2) * 4;
    return (ring > merge ? ring : merge) + 1024 + 256 + ATT_RECV_BYTES;
}

// 16 if this device co-schedules clusters of 16 CTAs of both decode kernels (opt-in), else 8.
int attn_max_cluster() {
    static int v = 0;
    if (v != 0) return v;
    v = 8;
    const char* env = getenv("GOGGUF_B200_ATTN_CLUSTER16");
    if (env != nullptr && env[0] == '0') return v;
    bool ok = true;
    auto probe = [&](auto kern, int smem) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
            cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) { ok = false; return; }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, 16);
        cfg.blockDim = dim3(160);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 16;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 8) ok = false;
    };
    probe(attn_decode_tma_kernel<128, 3>, decode_tma_smem<128, 3>());
    probe(attn_decode_tma_kernel<64, 4>, decode_tma_smem<64, 4>());
    cudaGetLastError();
    if (ok) v = 16;
    return v;
}

template <int D, int STAGES>
int launch_decode_tma(const CUtensorMap& tk, const CUtensorMap& tv, const void* q, void* out, float* part_o, float* part_ml,
                      const int* positions, const int* seq_of_token, const int* page_table, int max_pages, int ntok,
                      int nq, int nkv, float scale_log2, int window, int splits, bool cluster, int n_pages, int* status,
                      cudaStream_t stream) {
    constexpr int smem = decode_tma_smem<D, STAGES>();
    static bool configured = false;
    auto kern = attn_decode_tma_kernel<D, STAGES>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(ntok, nkv, splits);
    const int cl = (cluster && splits > 1) ? 1 : 0;
    static int places = 0;         // CTAs of this kernel that the device holds at once
    if (places == 0) {
        int dev = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 160, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
        places = (sms > 0 ? sms : 1) * per_sm;
    }
    const int early = (long long)ntok * nkv * splits <= places ? 1 : 0;
    return gg_launch(kern, grid, dim3(160), smem, stream, cl ? splits : 1, tk, tv, (const bf16*)q, (bf16*)out, part_o,
                     part_ml, positions, seq_of_token, page_table, max_pages, nq, nkv, scale_log2, window, splits, cl,
                     early, n_pages, status);
}


// ------------------------------------------------------------------------------------------- prefill, tcgen05
// Prefill attention on the 5th-generation tensor cores.  One CTA per (128-query tile of one sequence,
// query head).  Per 64-key page:  S = Q K^T  (tcgen05.mma 128 x 64 x 16, eight times; Q and K are
// K-major tiles staged by TMA) lands in tensor memory; the four softmax warps read it, one query row
// per thread, so the row maximum and sum need no exchange between threads; they write P as bfloat16
// back into tensor memory, over the first half of the score buffer it was made from (tcgen05.st), and
//  O += P V  (128 x D x 16, four times; P is the A operand straight from tensor memory, V the MN-major
// B operand in shared memory: one 128-byte row per key) accumulates in tensor memory.
// The maximum that P and the row sum are taken against is the one in use from the pages before (the result
// is exact whatever it is, as long as nothing overflows), so a page costs no pass over its scores for their
// maximum and no pass over O; only when the page's sum shows that a score lies more than 2^64 above it (or
// the row has no maximum yet) does the warp find the page's maximum, rescale O in place where it has grown
// by more than 2^8, and compute the page again.
// Two CTAs share an SM (96 KB of shared memory and 256 tensor-memory columns each): while one runs
// its softmax the other's MMAs keep the tensor pipe busy.
// All exponentials go to the special-function unit: computing a share of them as polynomials on the FMA pipe,
// and a pass over the scores for their maximum, cost more issue slots than the unit's time they saved.
template <int D>
__global__ void __launch_bounds__(192) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
    bf16* __restrict__ out, const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens,
    const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int max_pages, int n_seqs,
    int nq, int nkv, float scale_log2, int window, int n_pages, int* __restrict__ status) {
    constexpr int HALVES = D / 64;
    constexpr int QBOX = 128 * 64 * 2;              // [64 columns x 128 rows] box of Q: 16 KB
    constexpr int KBOX = 64 * 64 * 2;               // [64 columns x 64 rows] box of K or V: 8 KB
    constexpr int Q_BYTES = HALVES * QBOX, K_STAGE = HALVES * KBOX, V_BYTES = HALVES * KBOX;
    constexpr int TMEM_COLS = 256;
    // The dynamic segment is the only shared memory of this kernel and is asked to start on a 1024-byte
    // boundary (the swizzled tiles need it) instead of being rounded up in the kernel: two CTAs of 96.25 KB share an SM.
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* Qs = smem;
    uint8_t* Ks = Qs + Q_BYTES;                     // two stages
    // (a third stage of V in the place the P tile had was measured and changed nothing: 792 against 800 TFLOP/s
    // at 2,048 tokens, 1,118 against 1,125 at 8,192)
    constexpr int VST = 2;
    uint8_t* Vs = Ks + 2 * K_STAGE;                 // two stages
    uint64_t* bars = (uint64_t*)(Vs + 2 * V_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                    // [2]
    uint64_t* k_empty = bars + 3;                   // [2]
    uint64_t* v_full = bars + 5;                    // [3]
    uint64_t* v_empty = bars + 8;                   // [3]
    uint64_t* s_full = bars + 11;                   // [2]
    uint64_t* p_ready = bars + 13;
    uint64_t* pv_done = bars + 14;
    uint32_t* tmem_slot = (uint32_t*)(bars + 15);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    // no early release of the next kernel here: see the note on dependent launches in common.cuh
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        tma::mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) { tma::mbar_init(&k_full[i], 1); tma::mbar_init(&k_empty[i], 1); }
        for (int i = 0; i < 3; ++i) { tma::mbar_init(&v_full[i], 1); tma::mbar_init(&v_empty[i], 1); }
        tma::mbar_init(&s_full[0], 1); tma::mbar_init(&s_full[1], 1); tma::mbar_init(pv_done, 1);
        tma::mbar_init(p_ready, 4);           // one arrival per softmax warp
        *abort_flag = 0;
        tma::mbar_fence_init();
        tma::prefetch_map(&tmQ); tma::prefetch_map(&tmK); tma::prefetch_map(&tmV);
    }
    if (warp == 5) tc5::alloc(tmem_slot, TMEM_COLS);
    tc5::fence_before();
    __syncthreads();
    tc5::fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();          // q, the cache and the integer tables come from earlier kernels and copies

    // which (sequence, 128-row query tile)?  heavy tiles (late rows) first
    int b = -1, tile = (int)gridDim.y - 1 - (int)blockIdx.y, n_new = 0, tok0 = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const int a = cu_seqlens[i], e = cu_seqlens[i + 1];
        if (seq_of_token[a] < 0) continue;
        const int nt = (e - a + 127) >> 7;
        if (tile < nt) { b = i; n_new = e - a; tok0 = a; break; }
        tile -= nt;
    }
    // (a shared-memory base off the 1024-byte boundary would corrupt the swizzled tiles: refuse and say so)
    const bool aligned = (tma::smem_u32(smem) & 1023u) == 0;
    if (!aligned && threadIdx.x == 0) atomicCAS(status, 0, 29);
    const bool active = b >= 0 && aligned;
    const int h = blockIdx.x, kvh = active ? h / (nq / nkv) : 0;
    const int row0 = tile * 128;
    const int rows = active ? min(128, n_new - row0) : 0;
    const int pos0 = active ? ctx_lens[b] - n_new + row0 : 0;
    int lo = 0;
    if (window > 0 && pos0 - window + 1 > 0) lo = pos0 - window + 1;
    const int kt_first = lo / PAGE, kt_last = active ? (pos0 + rows - 1) / PAGE : -1;
    const int ntiles = kt_last - kt_first + 1;
    // tensor memory: two score buffers of 64 columns (the scores of page j + 1 are computed while the softmax
    // of page j runs), then the output accumulator
    const uint32_t S_t = tmem_base, O_t = tmem_base + 128;

    if (warp == 4) {
        if (lane == 0 && active) {
            const int* pt = page_table + (size_t)b * max_pages;
            tma::mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) tma::load_2d(Qs + hf * QBOX, &tmQ, q_full, h * D + hf * 64, tok0 + row0);
            for (int j = 0; j < ntiles; ++j) {
                const int s = j & 1;
                const int row = (gg_page(pt, kt_first + j, max_pages, PageBounds{n_pages, status}, 45) * nkv + kvh) * PAGE;
                if (!tma::mbar_wait(&k_empty[s], (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag, status, 21)) break;
                tma::mbar_expect_tx(&k_full[s], K_STAGE);
#pragma unroll
                for (int hf = 0; hf < HALVES; ++hf) tma::load_2d(Ks + s * K_STAGE + hf * KBOX, &tmK, &k_full[s], hf * 64, row);
                const int vs = j % VST;
                if (!tma::mbar_wait(&v_empty[vs], (uint32_t)((j / VST) & 1) ^ 1u, abort_flag, status, 22)) break;
                tma::mbar_expect_tx(&v_full[vs], V_BYTES);
#pragma unroll
                for (int hf = 0; hf < HALVES; ++hf) tma::load_2d(Vs + vs * V_BYTES + hf * KBOX, &tmV, &v_full[vs], hf * 64, row);
            }
        }
    } else if (warp == 5) {
        if (lane == 0 && active) {
            const uint32_t idesc_qk = tc5::idesc_bf16(128, 64, 0), idesc_pv = tc5::idesc_bf16(128, D, 1);
            const uint32_t q_a = tma::smem_u32(Qs), k_a = tma::smem_u32(Ks), v_a = tma::smem_u32(Vs);
            bool ok = tma::mbar_wait(q_full, 0, abort_flag, status, 23);
            // scores of page j into buffer j & 1
            auto issue_scores = [&](int j) -> bool {
                const int s = j & 1;
                if (!tma::mbar_wait(&k_full[s], (uint32_t)((j >> 1) & 1), abort_flag, status, 24)) return false;
                tc5::fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t a = tc5::smem_desc(q_a + (ks >> 2) * QBOX + (ks & 3) * 32, 16, 1024);
                    const uint64_t bb = tc5::smem_desc(k_a + s * K_STAGE + (ks >> 2) * KBOX + (ks & 3) * 32, 16, 1024);
                    tc5::mma(S_t + (uint32_t)(s * 64), a, bb, idesc_qk, ks > 0 ? 1u : 0u);
                }
                tc5::commit(&s_full[s]);
                tc5::commit(&k_empty[s]);
                return true;
            };
            if (ok && ntiles > 0) ok = issue_scores(0);
            for (int j = 0; j < ntiles && ok; ++j) {
                // The next page's scores do not wait for this page's softmax: their buffer was last read by the
                // softmax of page j - 1, whose p_ready this thread has already seen.
                if (j + 1 < ntiles) {
                    ok = issue_scores(j + 1);
                    if (!ok) break;
                }
                ok = tma::mbar_wait(p_ready, (uint32_t)(j & 1), abort_flag, status, 25);
                if (!ok) break;
                const int vs = j % VST;
                ok = tma::mbar_wait(&v_full[vs], (uint32_t)((j / VST) & 1), abort_flag, status, 26);
                if (!ok) break;
                tc5::fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t bb = tc5::smem_desc(v_a + vs * V_BYTES + kk * 2048, KBOX, 1024);
                    // P of page j lies in the first 32 columns of score buffer j & 1: 16 keys are 8 columns
                    tc5::mma_a_tmem(O_t, S_t + (uint32_t)((j & 1) * 64 + kk * 8), bb, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tc5::commit(pv_done);
                tc5::commit(&v_empty[vs]);
            }
        }
    } else if (active) {
        const int row = threadIdx.x;                       // query row of the tile = tensor-memory lane
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const int p = pos0 + row;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < ntiles; ++j) {
            if (!tma::mbar_wait(&s_full[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, status, 27)) { ok = false; break; }
            tc5::fence_after();
            uint32_t sr[64];
            tc5::ld32(S_t + lane_off + (uint32_t)((j & 1) * 64), sr);
            tc5::ld32(S_t + lane_off + (uint32_t)((j & 1) * 64) + 32, sr + 32);
            tc5::wait_ld();
            const int key0 = (kt_first + j) * PAGE;
            const bool edge = (key0 + PAGE - 1 > pos0) || (window > 0 && key0 < pos0 + 127 - window + 1);
            // masked keys become minus infinity (the scale is positive)
            if (edge) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int kidx = key0 + c;
                    bool vis = kidx <= p;
                    if (window > 0) vis = vis && (kidx > p - window);
                    if (!vis) sr[c] = 0xff800000u;
                }
            }
            uint32_t pk[32];
            // P = 2^(score * scale - maximum in use) as bfloat16 pairs; returns the sum of the page's P
            auto exponentials = [&]() -> float {
                const float mu = m_used == -INFINITY ? 0.f : m_used;
                const unsigned long long sc2 = pack2(scale_log2, scale_log2), nmu2 = pack2(-mu, -mu);
                unsigned long long l4[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    // exponent of the pair: score * scale - maximum in use, one packed multiply-add
                    float x0, x1, p0, p1;
                    unpack2(fma2(pack2(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1])), sc2, nmu2), x0, x1);
                    p0 = fast_exp2(x0);
                    p1 = fast_exp2(x1);
                    l4[e & 3] = add2(l4[e & 3], pack2(p0, p1));
                    pk[e] = pack_bf16(p0, p1);
                }
                float la, lb;
                unpack2(add2(add2(l4[0], l4[1]), add2(l4[2], l4[3])), la, lb);
                return la + lb;
            };
            // The maximum in use is stale on purpose: P and the row sum use the same one, so the result is exact
            // whatever it is, as long as nothing overflows.  So a page is first computed with the maximum of
            // the pages before it, without looking for its own; only when a row has no maximum yet, or the
            // page's sum says that a score lies more than 2^64 above it, the warp finds the page's maximum,
            // rescales O where it has grown by more than 2^8 and computes the page again.
            float lpage = 0.f;
            bool again = m_used == -INFINITY;
            if (!__any_sync(0xffffffffu, again)) {
                lpage = exponentials();
                again = !(lpage < 1.8446744e19f);
            }
            if (__any_sync(0xffffffffu, again)) {
                float mraw;
                {
                    // eight independent running maxima instead of one chain of 64 dependent operations
                    float m8[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) m8[k] = __uint_as_float(sr[k]);
#pragma unroll
                    for (int c = 8; c < 64; ++c) m8[c & 7] = fmaxf(m8[c & 7], __uint_as_float(sr[c]));
                    mraw = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
                }
                const float mx = mraw * scale_log2;
                const bool grow = mx > m_used + 8.0f || (m_used == -INFINITY && mx != -INFINITY);
                if (__any_sync(0xffffffffu, grow)) {
                    float corr = 1.0f;
                    if (grow) {
                        corr = m_used == -INFINITY ? 0.f : fast_exp2(m_used - mx);
                        m_used = mx;
                        l *= corr;
                    }
                    if (j > 0) {
                        // P V of the page before must be complete before O is rescaled
                        if (!tma::mbar_wait(pv_done, (uint32_t)((j - 1) & 1), abort_flag, status, 28)) { ok = false; break; }
                        tc5::fence_after();
#pragma unroll 1
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            uint32_t orow[32];
                            tc5::ld32(O_t + lane_off + c0, orow);
                            tc5::wait_ld();
#pragma unroll
                            for (int c = 0; c < 32; ++c) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * corr);
                            tc5::st32(O_t + lane_off + c0, orow);
                        }
                        tc5::wait_st();
                    }
                }
                lpage = exponentials();
            }
            l += lpage;
            // P over this thread's own row of the scores it has read (the first 32 of the buffer's 64 columns).
            // Nothing else uses this buffer now: the P V that read the P of two pages ago from it was issued
            // before the scores read above, and the tensor core works in order; the next scores into it are
            // issued after the P V that reads this P.  (The P V of the page before reads the other buffer; only
            // a rescaling of O has to wait for it.)
            tc5::st32(S_t + lane_off + (uint32_t)((j & 1) * 64), pk);
            tc5::wait_st();
            tc5::fence_before();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(p_ready);
        }
        // The last P V.  The scores of the last page say that the P V of two pages before is complete; the one
        // in between has not been waited for, and a wait by parity can only tell neighbouring phases apart.
        if (ok && ntiles > 1) ok = tma::mbar_wait(pv_done, (uint32_t)((ntiles - 2) & 1), abort_flag, status, 28);
        if (ok && tma::mbar_wait(pv_done, (uint32_t)((ntiles - 1) & 1), abort_flag, status, 28)) {
            tc5::fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = out + ((size_t)(tok0 + row0 + row) * nq + h) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t orow[32];
                tc5::ld32(O_t + lane_off + c0, orow);
                tc5::wait_ld();
                if (row < rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            pk[e] = pack_bf16(__uint_as_float(orow[c + 2 * e]) * inv, __uint_as_float(orow[c + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
        }
    }
    tc5::fence_before();
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
        __syncthreads();
    }
    if (warp == 5) {
        tc5::fence_after();
        tc5::dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace

// Number of key-range splits the decode launcher uses for this shape; the caller sizes the scratch:
// part_o needs ntok * nq * splits * d floats, part_ml ntok * nq * splits * 2 floats (when splits > 1).
GG_API gg_attn_decode_splits(int ntok, int nkv, int max_ctx) {
    if (ntok <= 0 || nkv <= 0) return 1;
    long long ctas = (long long)ntok * nkv;
    int splits = (int)((592 + ctas - 1) / ctas);          // about four CTAs per SM on 148 SMs
    const int most = max_ctx / 128 > 0 ? max_ctx / 128 : 1;  // at least 128 keys per split
    if (splits > most) splits = most;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    return splits;
}

// Decode-style attention: every token row is one query position (its own sequence row b, position
// positions[tok]).  q, out: [ntok, nq, d] bf16; pools [page][nkv][64][d] bf16.  d must be 64 or 128,
// nq / nkv at most 16, page size 64.  splits must be what gg_attn_decode_splits returned.
GG_API gg_attn_decode(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_o, float* part_ml,
                      const int* positions, const int* seq_of_token, const int* page_table, int max_pages,
                      int page_size, int n_pages, int ntok, int nq, int nkv, int d, float scale, int window, int splits,
                      int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (page_size != PAGE || nq <= 0 || nkv <= 0 || nq % nkv || nq / nkv > 16 || (d != 64 && d != 128) || splits < 1 ||
        nkv > 65535 || splits > 65535)
        return GG_ERR_ARG;
    if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return GG_ERR_ARG;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(ntok, nkv, splits);
    if (d == 128)
        gg_launch(attn_decode_kernel<128>, dim3(grid), dim3(128), 0, stream, 1, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out,
                                                          part_o, part_ml, positions, seq_of_token, page_table, max_pages,
                                                          nq, nkv, scale_log2, window, splits, PageBounds{n_pages, status});
    else
        gg_launch(attn_decode_kernel<64>, dim3(grid), dim3(128), 0, stream, 1, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out,
                                                         part_o, part_ml, positions, seq_of_token, page_table, max_pages,
                                                         nq, nkv, scale_log2, window, splits, PageBounds{n_pages, status});
    int rc = gg_last_error();
    if (rc != 0 || splits == 1) return rc;
    if (d == 128) gg_launch(attn_combine_kernel<128>, dim3(ntok * nq), dim3(128), 0, stream, 1, part_o, part_ml, (bf16*)out, splits);
    else gg_launch(attn_combine_kernel<64>, dim3(ntok * nq), dim3(64), 0, stream, 1, part_o, part_ml, (bf16*)out, splits);
    return gg_last_error();
}

// Prefill attention for a ragged batch: sequence i brings tokens cu_seqlens[i]..cu_seqlens[i+1]-1, whose
// absolute positions end at ctx_lens[i]-1.  max_tiles >= sum over sequences of ceil(new tokens / 64).
GG_API gg_attn_prefill(const void* q, const void* k_pool, const void* v_pool, void* out, const int* cu_seqlens,
                       const int* ctx_lens, const int* seq_of_token, const int* page_table, int max_pages,
                       int page_size, int n_pages, int n_seqs, int max_tiles, int nq, int nkv, int d, float scale,
                       int window, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_tiles <= 0) return 0;
    if (page_size != PAGE || nq <= 0 || nkv <= 0 || nq % nkv || (d != 64 && d != 128) || nq > 65535) return GG_ERR_ARG;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(max_tiles, nq);
    const int smem = 5 * 64 * d * 2;
    cudaError_t e;
    if (d == 128) {
        static bool cfg128 = false;
        if (!cfg128) {
            e = cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return (int)e;
            cfg128 = true;
        }
        gg_launch(attn_prefill_kernel<128>, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out,
                                                              cu_seqlens, ctx_lens, seq_of_token, page_table, max_pages, n_seqs,
                                                              nq, nkv, scale_log2, window, PageBounds{n_pages, status});
    } else {
        gg_launch(attn_prefill_kernel<64>, dim3(grid), dim3(128), smem, stream, 1, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out,
                                                             cu_seqlens, ctx_lens, seq_of_token, page_table, max_pages, n_seqs,
                                                             nq, nkv, scale_log2, window, PageBounds{n_pages, status});
    }
    return gg_last_error();
}

// Splits for the TMA form: whole pages per CTA.  use_cluster != 0: the splits of one (token, kv head)
// form a thread-block cluster (at most 8) and are merged through distributed shared memory; no scratch.
GG_API gg_attn_decode_tma_splits(int ntok, int nkv, int max_ctx, int use_cluster) {
    if (ntok <= 0 || nkv <= 0) return 1;
    const long long pairs = (long long)ntok * nkv;
    // cluster form: one wave of CTAs (two share an SM: 296 places); scratch form: about four waves
    int splits = use_cluster ? (int)(296 / pairs) : (int)((4 * 296 + pairs - 1) / pairs);
    const int pages = (max_ctx + PAGE - 1) / PAGE;
    if (splits > pages / 2) splits = pages / 2;       // at least two pages per CTA
    // Clusters of 16 (where the device takes them) pay off for the fewest sequences and long contexts only
    // (measured: 28 against 41 us for one sequence at 32K positions; slower than 8 from two sequences on).
    int most = 64;
    if (use_cluster) most = (pairs * 16 <= 148 && pages >= 64) ? attn_max_cluster() : 8;
    if (splits > most) splits = most;
    if (splits < 1) splits = 1;
    if (use_cluster) {
        // powers of two only: clusters of 5, 6, 7 or 12 CTAs ran 30-50 % slower than the next smaller power
        int p = 1;
        while (p * 2 <= splits) p *= 2;
        splits = p;
    }
    return splits;
}

// As gg_attn_decode, with the cache streamed by TMA.  n_pages is the number of pages in the pools
// (their first dimension); splits must be what gg_attn_decode_tma_splits returned for the same
// use_cluster; status as in the tensor-core product (codes 11 producer, 12 consumer).
GG_API gg_attn_decode_tma(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_o, float* part_ml,
                          const int* positions, const int* seq_of_token, const int* page_table, int max_pages,
                          int page_size, int n_pages, int ntok, int nq, int nkv, int d, float scale, int window,
                          int splits, int use_cluster, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (page_size != PAGE || nq <= 0 || nkv <= 0 || nq % nkv || nq / nkv > 16 || (d != 64 && d != 128) || splits < 1 ||
        nkv > 65535 || splits > 65535 || n_pages <= 0 || status == nullptr)
        return GG_ERR_ARG;
    const bool cluster = use_cluster != 0;
    if (cluster && splits > attn_max_cluster()) return GG_ERR_ARG;
    if (splits > 1 && !cluster && (part_o == nullptr || part_ml == nullptr)) return GG_ERR_ARG;
    if ((((uintptr_t)k_pool) & 15) || (((uintptr_t)v_pool) & 15)) return GG_ERR_ARG;
    CUtensorMap tk, tv;
    const unsigned long long rows = (unsigned long long)n_pages * nkv * PAGE;
    int rc;
    if ((rc = tma::make_map_bf16(&tk, k_pool, rows, d, d, PAGE)) != 0) return rc;
    if ((rc = tma::make_map_bf16(&tv, v_pool, rows, d, d, PAGE)) != 0) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    if (d == 128)
        rc = launch_decode_tma<128, 3>(tk, tv, q, out, part_o, part_ml, positions, seq_of_token, page_table, max_pages, ntok,
                                       nq, nkv, scale_log2, window, splits, cluster, n_pages, status, stream);
    else
        rc = launch_decode_tma<64, 4>(tk, tv, q, out, part_o, part_ml, positions, seq_of_token, page_table, max_pages, ntok,
                                      nq, nkv, scale_log2, window, splits, cluster, n_pages, status, stream);
    if (rc != 0 || splits == 1 || cluster) return rc;
    if (d == 128) gg_launch(attn_combine_kernel<128>, dim3(ntok * nq), dim3(128), 0, stream, 1, part_o, part_ml, (bf16*)out, splits);
    else gg_launch(attn_combine_kernel<64>, dim3(ntok * nq), dim3(64), 0, stream, 1, part_o, part_ml, (bf16*)out, splits);
    return gg_last_error();
}

// Prefill attention on tcgen05 (see attn_prefill_tc_kernel).  q and out: [n_tokens, nq, d] bf16, d = 64 or 128;
// pools [page][nkv][64][d]; max_tiles >= sum over sequences of ceil(new tokens / 128); status as in the
// tensor-core product (codes 21-28 name the wait that ran out).
GG_API gg_attn_prefill_tc(const void* q, const void* k_pool, const void* v_pool, void* out, const int* cu_seqlens,
                          const int* ctx_lens, const int* seq_of_token, const int* page_table, int max_pages,
                          int page_size, int n_pages, int n_tokens, int n_seqs, int max_tiles, int nq, int nkv, int d,
                          float scale, int window, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_tiles <= 0 || n_tokens <= 0) return 0;
    if (page_size != PAGE || nq <= 0 || nkv <= 0 || nq % nkv || (d != 64 && d != 128) || nq > 65535 || max_tiles > 65535 ||
        n_pages <= 0 || status == nullptr)
        return GG_ERR_ARG;
    if ((((uintptr_t)q) & 15) || (((uintptr_t)k_pool) & 15) || (((uintptr_t)v_pool) & 15) || (((uintptr_t)out) & 15)) return GG_ERR_ARG;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = tma::make_map_bf16(&tq, q, (unsigned long long)n_tokens, nq * d, (long long)nq * d, 128)) != 0) return rc;
    const unsigned long long rows = (unsigned long long)n_pages * nkv * PAGE;
    if ((rc = tma::make_map_bf16(&tk, k_pool, rows, d, d, PAGE)) != 0) return rc;
    if ((rc = tma::make_map_bf16(&tv, v_pool, rows, d, d, PAGE)) != 0) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(nq, max_tiles);
    if (d == 128) {
        constexpr int smem = 2 * 16384 + 2 * 16384 + 2 * 16384 + 256;   // Q, K x 2, V x 2, barriers
        static bool cfg = false;
        if (!cfg) {
            cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return (int)e;
            cfg = true;
        }
        return gg_launch(attn_prefill_tc_kernel<128>, grid, dim3(192), smem, stream, 1, tq, tk, tv, (bf16*)out, cu_seqlens,
                         ctx_lens, seq_of_token, page_table, max_pages, n_seqs, nq, nkv, scale_log2, window, n_pages, status);
    }
    constexpr int smem = 16384 + 2 * 8192 + 2 * 8192 + 256;
    static bool cfg64 = false;
    if (!cfg64) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        cfg64 = true;
    }
    return gg_launch(attn_prefill_tc_kernel<64>, grid, dim3(192), smem, stream, 1, tq, tk, tv, (bf16*)out, cu_seqlens,
                     ctx_lens, seq_of_token, page_table, max_pages, n_seqs, nq, nkv, scale_log2, window, n_pages, status);
}

// 1 if this library was built with checked page tables (the debug build), else 0.
GG_API gg_attention_fast_checked() { return gg_debug_bounds(); }
