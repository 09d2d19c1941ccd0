// MLA decode attention in latent space on CUDA cores (f32 accumulate):
//     out_h = sum_t softmax_t((q_h . [L_t | R_t]) * scale) * L_t
//
//   rivoli_mla_attend             : the reference operator (f32 q, fp8 latent slab with
//                                   per-128 block scales, bf16 roped keys, one sequence;
//                                   crates/backend/kernels/attn.hip:119-308).
//   rivoli_attend_simt_paged_bf16 : the same arithmetic on the paged fp8 pool (bf16 q,
//                                   one scale per token, fp8 roped keys), batched. This is the
//                                   f32 cross-check of the tensor-core kernel and the path
//                                   used for geometries that kernel does not cover.
//
// One CTA attends a GROUP of heads of one (sequence, split) - all of them whenever their q rows fit
// shared memory, otherwise groups tiled over gridDim.z - so each cached row is read from HBM once per
// (split, head group) (the reference re-reads it ceil(H/16) times). q sits in shared memory as f32
// for the whole CTA; rows are dequantised 16 at a time into a shared tile; warp w owns heads
// w, w + n_warps, ... of the group and its lanes own the columns i = lane (mod 32), so the online
// accumulator is lane-private registers.
#include "codec.cuh"
#include "common.cuh"

constexpr int AT_THREADS = 1024;
constexpr int AT_WARPS = 32;
constexpr int AT_TT = 16;          // rows per staged tile
constexpr int AT_MAX_SPLITS = 16;  // bounds the caller's scratch (attn.hip:67)

struct AttSlab {
    const float* qabs; const float* qrope; const unsigned char* lc8; const float* lscale;
    const unsigned short* rc; const unsigned int* rows; int n_blocks; float* clat;
};
struct AttPaged {
    const uint16_t* q; const uint8_t* pool; const float* pscale; const int32_t* block_table;
    const uint32_t* rows; long long row_stride; const int32_t* n_rows; int page_tokens; int max_pages;
    int n_pool_pages; uint16_t* out; float* out_m; float* out_lse;
    int rows_lo, rows_hi;   // the launch serves sequences with rows_lo <= n_rows < rows_hi only (others are left untouched)
};

template <bool PAGED, int HPW>
__global__ void __launch_bounds__(AT_THREADS, 1)
attend_simt_kernel(AttSlab sp, AttPaged pp, int H, int hg, int kvl, int rope, float scale, int nr_single,
                   int n_splits, float* __restrict__ partial) {
    extern __shared__ __align__(16) float smem[];
    const int W = kvl + rope;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int head0 = blockIdx.z * hg;             // this CTA's head group: [head0, head0 + Hc)
    const int Hc = min(hg, H - head0);
    float* qs = smem;                      // [hg][W]
    float* tile = smem + (size_t)hg * W;   // [AT_TT][W]
    __shared__ float tscale[AT_TT];
    __shared__ const uint8_t* trow[AT_TT];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, b = blockIdx.y;
    int nr = nr_single;
    if (PAGED) {  // clamp device-side counts so a bad entry can never index past a table
        rv_grid_dep_trigger();             // a dependent kernel may set itself up; it waits for this grid before reading
        rv_grid_dep_wait();                // the counts (and rows) may come from the kernel before
        nr = pp.n_rows[b];
        // a row list whose first entry is the dense marker stands for "row j = token j" over the first n_rows tokens
        if (pp.rows && pp.rows[(size_t)b * pp.row_stride] == 0xffffffffu) pp.rows = nullptr;
        const long long cap = pp.rows ? pp.row_stride : (long long)pp.max_pages * pp.page_tokens;
        nr = (int)max(0LL, min((long long)nr, cap));
        if (nr < pp.rows_lo || nr >= pp.rows_hi) return;   // another kernel of the same call serves this sequence
    }
    const int nacc = kvl / 32;             // lane-owned latent columns (<= 16)
    const int nrp = (rope + 31) / 32;      // lane-owned rope columns (<= 4)

    // q -> shared f32
    if (PAGED) {
        const uint16_t* q = pp.q + ((size_t)b * H + head0) * W;
        for (int i = tid; i < Hc * W; i += nthreads) qs[i] = rv_bf16_to_f32(q[i]);
    } else {
        for (int i = tid; i < Hc * W; i += nthreads) {
            const int h = i / W, c = i - h * W;
            qs[i] = c < kvl ? sp.qabs[(size_t)(head0 + h) * kvl + c] : sp.qrope[(size_t)(head0 + h) * rope + (c - kvl)];
        }
    }

    // this split's row range, tile aligned
    const int ntiles = (nr + AT_TT - 1) / AT_TT;
    const int tps = (ntiles + n_splits - 1) / n_splits;
    const int r_begin = split * tps * AT_TT;
    const int r_end = min(nr, r_begin + tps * AT_TT);

    float acc[HPW][16];
    float m[HPW], l[HPW];
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        m[j] = -INFINITY; l[j] = 0.0f;
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[j][k] = 0.0f;
    }

    for (int t0 = r_begin; t0 < r_end; t0 += AT_TT) {
        const int tcount = min(AT_TT, r_end - t0);
        __syncthreads();  // previous tile consumed (and q staged, first time round)
        if (PAGED) {
            if (tid < tcount) {
                const uint32_t t = pp.rows ? pp.rows[(size_t)b * pp.row_stride + t0 + tid] : (uint32_t)(t0 + tid);
                const int lp = (int)(t / (uint32_t)pp.page_tokens);
                int page = lp < pp.max_pages ? pp.block_table[(size_t)b * pp.max_pages + lp] : -1;
                if (page < 0 || page >= pp.n_pool_pages) page = 0;  // guarded: never read outside the pool
                const size_t r = (size_t)page * pp.page_tokens + (t & (uint32_t)(pp.page_tokens - 1));
                trow[tid] = pp.pool + r * W;
                tscale[tid] = pp.pscale[r];
            }
            __syncthreads();
            const int cpr = W / 16;  // 16-byte chunks per row
            for (int c = tid; c < tcount * cpr; c += nthreads) {
                const int row = c / cpr, ch = c - row * cpr;
                const uint4 p = *reinterpret_cast<const uint4*>(trow[row] + ch * 16);
                const float sc = tscale[row];
                const uint32_t wv[4] = {p.x, p.y, p.z, p.w};
                float* dst = tile + (size_t)row * W + ch * 16;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 a = rv_e4m3x2_to_f32x2((uint16_t)(wv[k] & 0xffff));
                    const float2 c2 = rv_e4m3x2_to_f32x2((uint16_t)(wv[k] >> 16));
                    dst[4 * k + 0] = __fmul_rn(a.x, sc); dst[4 * k + 1] = __fmul_rn(a.y, sc);
                    dst[4 * k + 2] = __fmul_rn(c2.x, sc); dst[4 * k + 3] = __fmul_rn(c2.y, sc);
                }
            }
        } else {
            for (int idx = tid; idx < tcount * W; idx += nthreads) {
                const int row = idx / W, c = idx - row * W;
                const size_t t = sp.rows ? (size_t)sp.rows[t0 + row] : (size_t)(t0 + row);
                tile[idx] = c < kvl
                    ? __fmul_rn(rv_e4m3_to_f32(sp.lc8[t * kvl + c]), sp.lscale[t * sp.n_blocks + c / 128])
                    : rv_bf16_to_f32(sp.rc[t * rope + (c - kvl)]);
            }
        }
        __syncthreads();

        for (int tt = 0; tt < tcount; ++tt) {
            const float* row = tile + (size_t)tt * W;
            float lv[16], rv[4];
#pragma unroll
            for (int k = 0; k < 16; ++k) lv[k] = k < nacc ? row[lane + 32 * k] : 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) rv[k] = (k < nrp && lane + 32 * k < rope) ? row[kvl + lane + 32 * k] : 0.0f;
#pragma unroll
            for (int j = 0; j < HPW; ++j) {
                const int hl = warp + nwarps * j;        // head within the group
                if (hl >= Hc) continue;                  // warp-uniform
                const float* qh = qs + (size_t)hl * W;
                float part = 0.0f;
#pragma unroll
                for (int k = 0; k < 16; ++k) if (k < nacc) part = fmaf(qh[lane + 32 * k], lv[k], part);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (k < nrp && lane + 32 * k < rope) part = fmaf(qh[kvl + lane + 32 * k], rv[k], part);
                const float s = rv_warp_sum(part) * scale;
                const float m_new = fmaxf(m[j], s);
                const float corr = expf(m[j] - m_new);
                const float p = expf(s - m_new);
#pragma unroll
                for (int k = 0; k < 16; ++k) acc[j][k] = fmaf(p, lv[k], acc[j][k] * corr);
                l[j] = fmaf(l[j], corr, p);
                m[j] = m_new;
            }
        }
    }

#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        if (warp + nwarps * j >= Hc) continue;
        const int head = head0 + warp + nwarps * j;
        if (n_splits > 1) {
            // unnormalised partial + (m, l); an empty split stores (-inf, 0, 0)
            float* base = partial + (size_t)b * n_splits * H * (kvl + 2);
            float* pa = base + ((size_t)split * H + head) * kvl;
            float* pml = base + (size_t)n_splits * H * kvl + ((size_t)split * H + head) * 2;
#pragma unroll
            for (int k = 0; k < 16; ++k) if (k < nacc) pa[lane + 32 * k] = acc[j][k];
            if (lane == 0) { pml[0] = m[j]; pml[1] = l[j]; }
        } else {
            const float inv = l[j] > 0.0f ? 1.0f / l[j] : 0.0f;
            if (PAGED) {
                uint16_t* o = pp.out + ((size_t)b * H + head) * kvl;
#pragma unroll
                for (int k = 0; k < 16; ++k) if (k < nacc) o[lane + 32 * k] = rv_f32_to_bf16(acc[j][k] * inv);
                if (lane == 0) {
                    if (pp.out_m) pp.out_m[(size_t)b * H + head] = m[j];
                    if (pp.out_lse) pp.out_lse[(size_t)b * H + head] = l[j] > 0.0f ? m[j] + logf(l[j]) : -INFINITY;
                }
            } else {
#pragma unroll
                for (int k = 0; k < 16; ++k) if (k < nacc) sp.clat[(size_t)head * kvl + lane + 32 * k] = acc[j][k] * inv;
            }
        }
    }
}

// Merge the split partials of one (sequence, head): w_s = exp(m_s - m_g), ascending split
// order (crates/backend/kernels/attn.hip:241-273).
template <bool PAGED>
__global__ void __launch_bounds__(128)
attend_combine_kernel(const float* __restrict__ partial, int H, int kvl, int n_splits, float* __restrict__ clat,
                      uint16_t* __restrict__ out, float* __restrict__ out_m, float* __restrict__ out_lse,
                      const int32_t* __restrict__ n_rows, long long cap, int rows_lo, int rows_hi, int serve_empty,
                      const uint32_t* __restrict__ rows, long long row_stride, long long dense_cap) {
    __shared__ float w[AT_MAX_SPLITS];
    __shared__ float inv_l;
    const int head = blockIdx.x, b = blockIdx.y;
    if (PAGED && n_rows) {   // same clamp and range rule as the kernels that wrote the partials
        if (rows && rows[(size_t)b * row_stride] == 0xffffffffu) cap = dense_cap;   // dense marker: see the attention kernels
        const int nr = (int)max(0LL, min((long long)n_rows[b], cap));
        if ((nr < rows_lo || nr >= rows_hi) && !(nr == 0 && serve_empty)) return;
    }
    const float* base = partial + (size_t)b * n_splits * H * (kvl + 2);
    const float* ml = base + (size_t)n_splits * H * kvl;
    if (threadIdx.x == 0) {
        float m_g = -INFINITY;
        for (int s = 0; s < n_splits; ++s) m_g = fmaxf(m_g, ml[((size_t)s * H + head) * 2]);
        float l_g = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float* p = ml + ((size_t)s * H + head) * 2;
            w[s] = isfinite(m_g) ? expf(p[0] - m_g) : 0.0f;
            l_g += p[1] * w[s];
        }
        inv_l = l_g > 0.0f ? 1.0f / l_g : 0.0f;
        if (PAGED) {
            if (out_m) out_m[(size_t)b * H + head] = m_g;
            if (out_lse) out_lse[(size_t)b * H + head] = l_g > 0.0f ? m_g + logf(l_g) : -INFINITY;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kvl; i += blockDim.x) {
        float sum = 0.0f;
        for (int s = 0; s < n_splits; ++s) sum += base[((size_t)s * H + head) * kvl + i] * w[s];
        if (PAGED) out[((size_t)b * H + head) * kvl + i] = rv_f32_to_bf16(sum * inv_l);
        else clat[(size_t)head * kvl + i] = sum * inv_l;
    }
}

// Launch plan: a CTA takes `hg` heads - all H when their q rows fit shared memory beside the row tile,
// otherwise (or when `hg_req` asks for smaller groups) H is tiled over gridDim.z - with one warp per head up
// to 32 warps, then 2 or 4 heads per warp. `dependent` launches the kernel as a programmatic dependent of the
// kernel before it in the stream (paged form only: it waits for that kernel before reading the counts).
template <bool PAGED>
static int launch_attend_simt(const AttSlab& sp, const AttPaged& pp, int H, int kvl, int rope, float scale,
                              int nr_single, int B, int n_splits, float* partial, cudaStream_t st, int hg_req = 0,
                              bool dependent = false) {
    const int W = kvl + rope;
    auto smem_of = [&](int h) { return ((size_t)h * W + (size_t)AT_TT * W) * sizeof(float); };
    const size_t smem_max = 227 * 1024 - 512;
    int hg = (hg_req > 0 && hg_req < H) ? hg_req : H;
    while (hg > 1 && (hg > 4 * AT_WARPS || smem_of(hg) > smem_max)) hg = (hg + 1) / 2;
    if (smem_of(hg) > smem_max) return 1006;
    const size_t smem = smem_of(hg);
    const int groups = (H + hg - 1) / hg;
    const int warps = hg < AT_WARPS ? hg : AT_WARPS;
    const int hpw = (hg + warps - 1) / warps;
    dim3 grid(n_splits, B, groups);
    rv_drain_error();
#define RV_ATT(HPW)                                                                                       \
    do {                                                                                                  \
        cudaFuncSetAttribute(attend_simt_kernel<PAGED, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             (int)smem);                                                                  \
        if (dependent)                                                                                    \
            rv_launch_dependent(attend_simt_kernel<PAGED, HPW>, grid, dim3(warps * 32), smem, st, sp, pp, H, hg, kvl,  \
                                rope, scale, nr_single, n_splits, partial);                               \
        else                                                                                              \
            attend_simt_kernel<PAGED, HPW><<<grid, warps * 32, smem, st>>>(sp, pp, H, hg, kvl, rope, scale, \
                                                                          nr_single, n_splits, partial);  \
    } while (0)
    if (hpw <= 1) RV_ATT(1);
    else if (hpw <= 2) RV_ATT(2);
    else RV_ATT(4);
#undef RV_ATT
    int e = rv_launch_status();
    if (e || n_splits <= 1) return e;
    const long long cap = PAGED ? (pp.rows ? pp.row_stride : (long long)pp.max_pages * pp.page_tokens) : 0;
    attend_combine_kernel<PAGED><<<dim3(H, B), 128, 0, st>>>(partial, H, kvl, n_splits, sp.clat, pp.out,
                                                              pp.out_m, pp.out_lse, PAGED ? pp.n_rows : nullptr, cap,
                                                              pp.rows_lo, pp.rows_hi, 0, pp.rows, pp.row_stride,
                                                              (long long)pp.max_pages * pp.page_tokens);
    return rv_launch_status();
}

// Combine launcher shared with the tensor-core kernel (same partial layout). Sequences whose row count
// lies outside [rows_lo, rows_hi) are left untouched (another kernel of the same call wrote them), except
// that an empty sequence is served when serve_empty is set.
extern "C" void rivoli_attend_combine_paged(const float* partial, int H, int kvl, int n_splits, int B, uint16_t* out,
                                            float* out_m, float* out_lse, const int32_t* n_rows, long long cap,
                                            int rows_lo, int rows_hi, int serve_empty, const uint32_t* rows,
                                            long long row_stride, long long dense_cap, cudaStream_t st) {
    attend_combine_kernel<true><<<dim3(H, B), 128, 0, st>>>(partial, H, kvl, n_splits, nullptr, out, out_m, out_lse,
                                                            n_rows, cap, rows_lo, rows_hi, serve_empty, rows, row_stride,
                                                            dense_cap);
}

RIVOLI_API size_t rivoli_mla_attend_scratch_floats(int H, int kvl) {
    if (H <= 0 || kvl <= 0) return 0;
    return (size_t)AT_MAX_SPLITS * (size_t)H * ((size_t)kvl + 2);
}

RIVOLI_API int rivoli_mla_attend(const float* qabs, const float* qrope, const unsigned char* Lc8,
                                 const float* Lscale, const unsigned short* Rc, const unsigned int* rows,
                                 int H, int nr, int kvl, int rope, int n_blocks, float scale, float* clat,
                                 float* partial) {
    if (H <= 0 || nr <= 0 || kvl <= 0 || rope <= 0 || n_blocks <= 0) return 1001;
    // The reference's staging bound and width rule, kept so the same shapes are rejected
    // with the same codes (attn.hip:285-293).
    if (((size_t)16 * kvl + (size_t)16 * rope) * sizeof(float) > 65536) return 1002;
    if (kvl > 512 || (kvl % 128) != 0) return 1004;
    if (rope > 128) return 1002;
    // Any H: heads beyond what one CTA's shared memory holds are tiled over gridDim.z (the reference tiles
    // them in blocks of 16, attn.hip:119-130). Split plan: a pure function of (H, nr, scratch present) ->
    // same shape, same summation order.
    int n_splits = 1;
    if (partial) {
        n_splits = (nr + 255) / 256;
        if (n_splits > AT_MAX_SPLITS) n_splits = AT_MAX_SPLITS;
        if (n_splits < 1) n_splits = 1;
    }
    AttSlab sp{qabs, qrope, Lc8, Lscale, Rc, rows, n_blocks, clat};
    AttPaged pp{};
    return launch_attend_simt<false>(sp, pp, H, kvl, rope, scale, nr, 1, n_splits, partial, 0);
}

// ------------------------------------------------------------------------------------------
// rivoli_mla_attend_static: rivoli_mla_attend for callers that have no device memory to lend.
//
// Some users of this library are not in a position to call cudaMalloc at all: an engine that
// carved up the whole device into its own arenas at start-up and treats any later driver
// allocation as a bug, a decode thread that must never block on the allocator (cudaMalloc
// and cudaFree serialise against the whole device), or a plugin host whose contract says
// the plugin owns no device memory. For them the split-KV partials that rivoli_mla_attend
// takes as the caller's `partial` scratch live here instead, in a fixed array inside the
// library image. It is sized for the model geometry only (H <= 64 heads, kvl <= 512):
// 16 splits x 64 x 514 floats = 2,105,344 bytes, which every GPU that loads this library
// carries until the process exits.
//
// The array's name is only a host-side handle for the symbol, never a device address, so the
// address is looked up once per device (with that device current) by cudaGetSymbolAddress
// and that pointer is what the kernels receive. The FIRST call on a device performs that
// look-up; make it before any stream capture begins on that device.
//
// All calls share the one array and it keeps whatever the last call left there. Nothing
// in it has to start at zero (every split, an empty one included, stores its partial before
// the combine reads it), but two calls that are in flight on the GPU at the same time (two
// streams, or two host threads on one device) would overwrite each other's partials: keep
// calls on one device ordered. Runs on the legacy default stream like rivoli_mla_attend.
// ------------------------------------------------------------------------------------------
constexpr int NA_MAX_H = 64, NA_MAX_KVL = 512, NA_MAX_DEVICES = 64;
static __device__ __align__(256) float g_attend_static_partial[AT_MAX_SPLITS * NA_MAX_H * (NA_MAX_KVL + 2)];
static float* g_attend_static_ptr[NA_MAX_DEVICES];   // per-device address of the array above (host side)

RIVOLI_API int rivoli_mla_attend_static(const float* qabs, const float* qrope, const unsigned char* Lc8,
                                        const float* Lscale, const unsigned short* Rc, const unsigned int* rows,
                                        int H, int nr, int kvl, int rope, int n_blocks, float scale, float* clat) {
    if (H <= 0 || nr <= 0 || kvl <= 0 || rope <= 0 || n_blocks <= 0) return 1001;
    if (((size_t)16 * kvl + (size_t)16 * rope) * sizeof(float) > 65536) return 1002;
    if (kvl > 512 || (kvl % 128) != 0) return 1004;
    if (rope > 128) return 1002;
    if (H > NA_MAX_H || kvl > NA_MAX_KVL) return 1002;   // beyond the built-in scratch: use rivoli_mla_attend
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -(int)e;
    if (dev < 0 || dev >= NA_MAX_DEVICES) return 1008;
    if (!g_attend_static_ptr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_attend_static_partial);
        if (e != cudaSuccess) return -(int)e;
        g_attend_static_ptr[dev] = p;
    }
    int n_splits = (nr + 255) / 256;                    // same plan as rivoli_mla_attend with scratch
    if (n_splits > AT_MAX_SPLITS) n_splits = AT_MAX_SPLITS;
    if (n_splits < 1) n_splits = 1;
    AttSlab sp{qabs, qrope, Lc8, Lscale, Rc, rows, n_blocks, clat};
    AttPaged pp{};
    return launch_attend_simt<false>(sp, pp, H, kvl, rope, scale, nr, 1, n_splits, g_attend_static_ptr[dev], 0);
}

// Split count of the SIMT paged path: a pure function of the batch size.
static int simt_paged_splits(int B) {
    int n = (2 * 148 + B - 1) / B;
    if (n > AT_MAX_SPLITS) n = AT_MAX_SPLITS;
    if (n < 1) n = 1;
    return n;
}

RIVOLI_API size_t rivoli_attend_simt_scratch_bytes(const DsaGeom* g, int B) {
    if (!g || B <= 0) return 0;
    return (size_t)B * simt_paged_splits(B) * g->n_heads * ((size_t)g->kv_lora + 2) * sizeof(float);
}

// Paged bf16 attention on CUDA cores. Same contract as rivoli_mla_attend_paged_bf16.
RIVOLI_API int rivoli_attend_simt_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                             const float* latent_scale, const int32_t* block_table,
                                             const uint32_t* rows, int row_stride, const int32_t* n_rows,
                                             int B, uint16_t* out, float* out_m, float* out_lse,
                                             void* scratch, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || !q || !latent_pool || !latent_scale || !block_table || !n_rows || !out) return 1001;
    if (rows && row_stride <= 0) return 1001;
    if (((uintptr_t)latent_pool & 15) || ((g->kv_lora + g->rope_dim) % 16) != 0) return 1005;
    int n_splits = scratch ? simt_paged_splits(B) : 1;
    AttSlab sp{};
    AttPaged pp{q, latent_pool, latent_scale, block_table, rows, row_stride, n_rows, g->page_tokens,
                g->max_pages_per_seq, g->n_pool_pages, out, out_m, out_lse, 0, 0x7fffffff};
    return launch_attend_simt<true>(sp, pp, g->n_heads, g->kv_lora, g->rope_dim, g->softmax_scale, 0, B,
                                    n_splits, (float*)scratch, (cudaStream_t)stream);
}

// The sequences of a batch with 0 < n_rows < rows_hi, on the CUDA-core kernel, eight heads per CTA and no
// split (no scratch): the short-context arm of rivoli_mla_attend_paged_bf16, launched in front of the
// tensor-core kernel as a programmatic dependent of whatever precedes it in the stream.
extern "C" int rivoli_attend_simt_short_rows(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                             const float* latent_scale, const int32_t* block_table,
                                             const uint32_t* rows, int row_stride, const int32_t* n_rows, int B,
                                             uint16_t* out, float* out_m, float* out_lse, int rows_hi,
                                             cudaStream_t st) {
    AttSlab sp{};
    AttPaged pp{q, latent_pool, latent_scale, block_table, rows, row_stride, n_rows, g->page_tokens,
                g->max_pages_per_seq, g->n_pool_pages, out, out_m, out_lse, 1, rows_hi};
    return launch_attend_simt<true>(sp, pp, g->n_heads, g->kv_lora, g->rope_dim, g->softmax_scale, 0, B, 1, nullptr,
                                    st, 8, true);
}
