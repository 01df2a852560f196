// Tensor-core GEMM family for the SwiGLU MLP on sm_100a: tcgen05.mma with accumulators in tensor
// memory (TMEM), operands staged in shared memory by TMA, fused epilogues.
//
// Replaces, on the MLP hot path, the two library GEMMs and the Triton activation kernel of
// MegaGemmTriton.forward (megagemm/swiglu.py:166-169: w12(x) -> MegaGemmFunction -> w3(h)):
//   * mgr_swiglu_fused_fwd : h = silu(x Wg^T) * (x Wv^T) in ONE kernel; each CTA tile owns 128 gate
//     columns and the matching 128 value columns (two B boxes of w12: rows n0.. and F+n0..), so the
//     [M, 2F] projection never reaches HBM;
//   * mgr_gemm_tn          : C = A B^T (nn.Linear without bias), used for w3(h);
// and the four GEMMs autograd runs for the two nn.Linear layers in backward plus the Triton backward
// kernel (megagemm/swiglu.py:111-131):
//   * mgr_gemm              : C = op(A) op(B)^T with either operand stored K-major or MN-major, which
//     covers dh = dy W3, dW3 = dy^T h, dx = dGV W12 and dW12 = dGV^T x without any transposed copy;
//   * mgr_swiglu_fused_bwd  : recomputes the projection tile by tile and turns it, with the matching
//     dh tile, into [d_gate | d_val] in the epilogue -- the projection is not stored in forward.
//
// Kernel shape (one CTA per SM, persistent over output tiles, 320 threads):
//   warp 0    : TMA producer  -- cp.async.bulk.tensor.2d into a 4-stage ring (A 128x64, B 256x64, 128B swizzle)
//   warp 1    : MMA issuer    -- one elected thread issues tcgen05.mma (M128 N256 K16, fp32 accumulate);
//               also owns the TMEM allocation (512 columns = two 128x256 accumulators)
//   warps 2-9 : epilogue      -- tcgen05.ld the finished accumulator, apply the epilogue, store (two warps per
//               32-lane quarter of tensor memory, each taking half of the column chunks); the second
//               accumulator lets the next tile's main loop run meanwhile.
// Every CTA issues its own loads. Every mbarrier wait is bounded (mgr_ptx.cuh).

#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <type_traits>

#include "mgr_common.cuh"
#include "mgr_ptx.cuh"

namespace mgr {
namespace {

__device__ int g_gemm_status = 0;

constexpr int kBM = 128;         // tile rows (UMMA M)
constexpr int kBN = 256;         // accumulator columns per tile (UMMA N) of the throughput kernels
constexpr int kBNSmall = 64;     // ... of the narrow-tile kernels used when a problem has few tiles (skinny M)
constexpr int kBNTiny = 32;      // ... and of the narrowest ones, for problems that still leave SMs idle at 64
constexpr int kBNMid = 96;       // ... 48 gate + 48 value columns: the fused projection of a skinny batch whose 32-column
                                 // tiles would need two rounds over the SMs (hidden 6912: 216 tiles of 32 against 144 of 48)
constexpr int kBK = 64;          // K per stage: 64 x 2 B = one 128-byte swizzle row
constexpr int kUmmaK = 16;       // K of one tcgen05.mma for 16-bit operands
constexpr uint32_t kABytes = kBM * kBK * 2;   // 16 KB: this CTA's 128 rows of A
__host__ __device__ constexpr uint32_t b_bytes(int bn) { return bn * kBK * 2; }   // 32 KB at BN 256 (a CTA pair holds half each)
// CG = CTAs that share one MMA (tcgen05 cta_group): 1, or 2 = a pair of CTAs in one cluster working on a
// 256 x 256 tile, each loading its own A rows and HALF of the B rows, which halves the B traffic per CTA
// and deepens the ring from 4 to 7 stages.
__host__ __device__ constexpr uint32_t stage_bytes(int cg, int bn) { return kABytes + b_bytes(bn) / cg; }
__host__ __device__ constexpr int num_stages(int cg, int bn) { return bn < kBN ? 8 : (cg == 1 ? 4 : 7); }
// + slack to align to 1024 B. The narrow-tile kernels take (nearly) all the shared memory an SM has and cut it into
// as many stages as fit at run time (a short A box makes a stage smaller, see narrow_geom()).
constexpr uint32_t kNarrowRing = 216 * 1024;
__host__ __device__ constexpr uint32_t gemm_smem(int cg, int bn) {
    return (bn < kBN ? kNarrowRing : num_stages(cg, bn) * stage_bytes(cg, bn)) + 1024;
}
// The dh -> [d_gate | d_val] epilogue moves its global traffic (the stored projection in, the gradients out)
// in a coalesced layout and converts to and from the accumulator's row-per-thread layout through a small
// per-warp staging buffer behind the ring: 32 rows x 64 B. The four 16-byte pieces of row r sit at piece ^ ((r >> 1) & 3):
// with that, a quarter-warp touches eight different 16-byte slots of the 128 bank bytes both ways round (one row per
// lane, and four lanes per row), where rows padded to 80 B left the four-lanes-per-row accesses a two-way conflict.
constexpr uint32_t kEpiRowPitch = 64;
constexpr uint32_t kEpiStageBytes = 32 * kEpiRowPitch;
constexpr int kMaxStages = 8;
// Narrow-tile kernels: a sub-stage is the A box actually loaded (8..128 rows) plus the 8 KB B tile of one
// 64-element K block; a STAGE (one full/empty barrier pair) is `ksub` consecutive sub-stages, i.e. ksub K blocks
// requested together. A decode-sized batch is bound by streaming the weights once; 64-element K blocks handled
// one barrier round trip at a time held an SM to ~40 GB/s (each weight row was touched 128 bytes at a time, and
// every 8 KB paid a wait / issue / commit round). With ksub = 4 a stage asks for 512 contiguous bytes of each
// weight row at once and the fixed cost per stage is spread over 32 KB.
struct NarrowGeom {
    int ksub, stages;
    uint32_t sub_bytes;
};
__host__ __device__ constexpr NarrowGeom narrow_geom(uint32_t a_box_bytes, int bn) {
    NarrowGeom g{0, 0, 0};
    g.sub_bytes = a_box_bytes + b_bytes(bn);
    // The MMA reads a full 128-row A operand (16 KB from the sub-stage's start) whatever the box loaded; the rows
    // beyond the box only feed output rows that are never stored, but the read itself must stay inside the ring
    // (reading past the CTA's shared memory is an illegal access): the last sub-stage must end >= 16 KB before
    // the end of the ring.
    const uint32_t tail = kABytes > g.sub_bytes ? kABytes - g.sub_bytes : 0u;
    g.ksub = bn <= kBNTiny ? 8 : 4;
    while (g.ksub > 1 && (kNarrowRing - tail) / (g.ksub * g.sub_bytes) < 4) g.ksub >>= 1;   // keep >= 4 stages in flight
    const uint32_t n = (kNarrowRing - tail) / (g.ksub * g.sub_bytes);
    g.stages = n > static_cast<uint32_t>(kMaxStages) ? kMaxStages : static_cast<int>(n);
    return g;
}
// Checked at compile time for every A box (8..128 rows) and both narrow widths: at least two stages, the ring
// holds them, and the 16 KB A window of the very last sub-stage ends inside the ring.
constexpr bool narrow_geom_fits(int bn) {
    for (uint32_t rows = 8; rows <= static_cast<uint32_t>(kBM); rows += 8) {
        const NarrowGeom g = narrow_geom(rows * kBK * 2, bn);
        const uint32_t last_sub = (static_cast<uint32_t>(g.stages) * g.ksub - 1) * g.sub_bytes;
        if (g.stages < 2 || g.stages > kMaxStages || g.ksub < 1) return false;
        if (last_sub + kABytes > kNarrowRing || last_sub + g.sub_bytes > kNarrowRing) return false;
    }
    return true;
}
static_assert(narrow_geom_fits(kBNSmall) && narrow_geom_fits(kBNTiny) && narrow_geom_fits(kBNMid), "narrow-tile ring geometry leaves shared memory");

constexpr int kEpiWarps = 8;      // epilogue warps: two per 32-lane quarter of tensor memory
// ring depth and dynamic shared memory of a kernel instance (a CTA pair gives up one stage to the staging buffers)
__host__ __device__ constexpr int num_stages_epi(int epi, int cg, int bn) {
    return (epi == 4 && cg == 2) ? 6 : num_stages(cg, bn);
}
__host__ __device__ constexpr uint32_t gemm_smem_epi(int epi, int cg, int bn) {
    return epi == 4 ? num_stages_epi(epi, cg, bn) * stage_bytes(cg, bn) + 1024 + kEpiWarps * kEpiStageBytes : gemm_smem(cg, bn);
}
constexpr int kGemmThreads = (2 + kEpiWarps) * 32;
// Shared-memory budget of every kernel instance, checked at compile time: the dynamic ring (+ staging buffers)
// plus 2 KB for the static barriers and flags stays within the 227 KB a CTA may use; stages and staging rows keep
// the alignment the 128-byte swizzle (1024 B) and the 16-byte shared-memory vectors need.
constexpr bool smem_budgets_ok() {
    constexpr uint32_t kCtaLimit = 227u * 1024u, kStatic = 2048u;
    for (int epi = 0; epi <= 4; ++epi)
        for (int cg = 1; cg <= 2; ++cg) {
            if (gemm_smem_epi(epi, cg, kBN) + kStatic > kCtaLimit) return false;
            if (stage_bytes(cg, kBN) % 1024u != 0 || num_stages_epi(epi, cg, kBN) > kMaxStages) return false;
        }
    if (gemm_smem(1, kBNSmall) + kStatic > kCtaLimit || gemm_smem(1, kBNTiny) + kStatic > kCtaLimit || gemm_smem(1, kBNMid) + kStatic > kCtaLimit) return false;
    if ((b_bytes(kBNMid) / 2) % 1024u != 0) return false;   // the value half of a 96-column B tile starts on a swizzle-group boundary
    return kEpiRowPitch % 16u == 0 && kEpiStageBytes % 16u == 0 && kNarrowRing % 1024u == 0 && b_bytes(kBNTiny) % 1024u == 0;
}
static_assert(smem_budgets_ok(), "a GEMM kernel instance exceeds the shared-memory budget or breaks an alignment rule");
constexpr uint32_t kTmemCols = 512;

enum Epilogue { kEpiPlain = 0, kEpiSwiglu = 1, kEpiSwigluBwd = 2, kEpiSwigluSave = 3, kEpiDhDgv = 4 };

// Output columns one tile covers: the full 256-column accumulator, or 128 when the accumulator holds a
// gate half and a value half.
__host__ __device__ constexpr int n_step_of(int epi, int bn) { return (epi == kEpiPlain || epi == kEpiDhDgv) ? bn : bn / 2; }

// Shared-memory matrix descriptors (64-bit, addresses in 16-byte units): start address [0,14),
// leading byte offset [16,30), stride byte offset [32,46), descriptor version 1 at [46,48) (sm_100),
// layout type 2 = SWIZZLE_128B at [61,64). Both operand layouts are what TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B: rows of 128 bytes, swizzled in 1024-byte groups of 8 rows.
//   K-major  (operand stored [rows, K]):  a smem row is one operand row, 64 K-elements. 8-row groups are
//            1024 B apart (stride offset); the leading offset is unused for swizzled K-major (encoded 1).
//            The next K=16 slice starts 32 B further along the row.
//   MN-major (operand stored [K, rows]):  a smem row is one K index, 64 consecutive operand rows. The tile
//            is a sequence of 64-row chunks, each [64 K x 128 B] = 8192 B: leading offset = 8192 B between
//            chunks, stride offset = 1024 B between groups of 8 K indices. The next K=16 slice starts
//            16 rows = 2048 B further.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, bool mn_major) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>(mn_major ? (8192 >> 4) : 1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor, kind::f16: fp32 accumulator (bits [4,6) = 1), operand formats at [7,10) and
// [10,13) (0 = fp16, 1 = bf16), A / B major-ness at bits 15 / 16 (1 = MN-major), N>>3 at [17,23),
// M>>4 at [24,29). N=256; M=128, or 256 for a CTA pair.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, bool a_mn, bool b_mn, int cg, int bn) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn ? (1u << 15) : 0u) | (b_mn ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>((kBM * cg) >> 4) << 24);
}

// MUFU exp + MUFU reciprocal: about 2 ulp, far below the 16-bit output rounding; keeps the epilogue short
__device__ __forceinline__ float sigmoid_(float g) { return __fdividef(1.0f, 1.0f + __expf(-g)); }
__device__ __forceinline__ float silu_mul(float g, float v) { return (g * sigmoid_(g)) * v; }

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// C tile coordinates of linear tile index t. Tiles are walked in bands of kBandRows rows of C: inside a
// band the M index runs fastest, then N; then the next band. The CTAs running at one time therefore cover
// a roughly square patch of C (about 2048 rows x 2300 columns on 148 SMs), so the A rows and B rows they
// stream fit in L2 together and each is fetched from HBM about once per band instead of once per N tile
// (which is what an M-fastest walk over a tall C costs, e.g. dW12 with 16384 rows).
constexpr int kBandRows = 2048;
struct TileCoord {
    int m0, n0;
};
__host__ __device__ constexpr TileCoord tile_coord(int t, int m_tiles, int n_tiles, int n_step, int m_step) {
    const int band = kBandRows / m_step;                 // M tiles per band
    const int per_band = band * n_tiles;
    const int b = t / per_band;
    const int r = t - b * per_band;
    const int rows_here = m_tiles - b * band < band ? m_tiles - b * band : band;   // the last band may be short
    const int mi = b * band + r % rows_here;
    const int ni = r / rows_here;
    return TileCoord{mi * m_step, ni * n_step};
}
// Checked at compile time: the walk visits every tile of an m_tiles x n_tiles grid exactly once, for single CTAs
// (128-row steps, 16 row tiles per band) and pairs (256-row steps, 8 per band), full and short last bands -- up to
// 40 row tiles exhaustively, and at the row-tile counts of the 16384-token block (128 single / 64 paired) and
// their neighbours.
constexpr bool tile_walk_visits_each_tile_once(int m_tiles, int n_tiles, int m_step) {
    bool seen[136 * 16] = {};
    for (int t = 0; t < m_tiles * n_tiles; ++t) {
        const TileCoord c = tile_coord(t, m_tiles, n_tiles, kBN, m_step);
        if (c.m0 < 0 || c.n0 < 0 || c.m0 % m_step != 0 || c.n0 % kBN != 0) return false;
        const int mi = c.m0 / m_step, ni = c.n0 / kBN;
        if (mi >= m_tiles || ni >= n_tiles || seen[mi * 16 + ni]) return false;
        seen[mi * 16 + ni] = true;
    }
    return true;
}
constexpr bool tile_walks_ok() {
    const int steps[2] = {kBM, 2 * kBM};
    for (int s = 0; s < 2; ++s)
        for (int m = 1; m <= 40; ++m)
            for (int n = 1; n <= 13; n += 3)
                if (!tile_walk_visits_each_tile_once(m, n, steps[s])) return false;
    const int big[8] = {63, 64, 65, 96, 127, 128, 129, 136};
    for (int s = 0; s < 2; ++s)
        for (int i = 0; i < 8; ++i)
            for (int n = 1; n <= 15; n += 7)
                if (!tile_walk_visits_each_tile_once(big[i], n, steps[s])) return false;
    return true;
}
static_assert(tile_walks_ok(), "the band-wise tile walk skips or repeats a tile");

// C = op(A) op(B)^T on one 128 x 256 accumulator tile per step.
//   A: K-major = stored [M, K] (tmA box 64(K) x 128);  MN-major = stored [K, M] (tmA box 64(M) x 64(K)).
//   B: K-major = stored [Nb, K] (tmB box 64(K) x 128); MN-major = stored [K, Nb] (tmB box 64(N) x 64(K)).
// kEpiPlain    : C[M, n_out] = acc; a tile covers 256 columns of C (B rows n0 .. n0+255).
// kEpiSwiglu   : B K-major = [gate rows | value rows] of n_out rows each. C[M, n_out] = silu(G) * V; a tile
//                covers 128 columns of C (B rows n0.. and n_out+n0..). With row_scale != NULL both halves of row r
//                are multiplied by row_scale[r] first: G = s_r (x w_g^T), V = s_r (x w_v^T) -- an RMSNorm in front
//                of the projection whose weight has been folded into w12 (s_r = 1 / rms of row r).
// kEpiSwigluBwd: same tile; aux = dh [M, n_out]. C = [d_gate | d_val] of shape [M, 2 n_out]:
//                d_val = dh * G * sig(G), d_gate = dh * V * sig(G) * (1 + G * (1 - sig(G))).
// kEpiSwigluSave: kEpiSwiglu that also stores the projection, rounded to T, in C2 = [G | V] of shape
//                [M, 2 n_out] (pitch ld_aux) -- the training forward, whose backward reads it back.
// kEpiDhDgv    : plain tile (256 columns); acc = dh tile; aux = stored projection [G | V] (pitch ld_aux);
//                C = [d_gate | d_val] of shape [M, 2 n_out]. dh itself is never written.
template <int EPI, bool A_MN, bool B_MN, int CG, typename T, int BN = kBN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, T* __restrict__ C,
            T* __restrict__ C2, const T* __restrict__ aux, int M, int n_out, int K, int64_t ldc, int64_t ld_aux,
            uint32_t a_box_bytes, const float* __restrict__ row_scale,
            int* __restrict__ status) {
    static_assert(n_step_of(EPI, BN) == BN || !B_MN, "the gate/value split reads w12 K-major");
    static_assert(BN == kBN || ((BN == kBNSmall || BN == kBNTiny) && CG == 1 && !A_MN && !B_MN && (EPI == kEpiPlain || EPI == kEpiSwiglu)) ||
                      (BN == kBNMid && CG == 1 && !A_MN && !B_MN && EPI == kEpiSwiglu),
                  "narrow tiles: single CTA, K-major operands, plain or fused-activation epilogue (96 columns: the latter only)");
    constexpr int kNStep = n_step_of(EPI, BN);  // output columns per tile
    // tensor-memory columns from one accumulator to the next: the tile width, rounded up to 128 for the 96-column tile
    // (whose second 32-column read of each half runs past column 96 and must not reach the other accumulator)
    constexpr int kAccStride = BN == kBNMid ? 128 : BN;
    // 32-column chunks of the tile's output an epilogue warp pair walks (the 16-column tile has a path of its own)
    constexpr int kChunks = kNStep < 32 ? 0 : (kNStep + 31) / 32;
    constexpr uint32_t kBBytes = b_bytes(BN);
    constexpr bool kNarrow = BN < kBN;
    // wide tiles: compile-time ring of one K block per stage; narrow tiles: see narrow_geom()
    const NarrowGeom ng = kNarrow ? narrow_geom(a_box_bytes, BN) : NarrowGeom{1, num_stages_epi(EPI, CG, BN), stage_bytes(CG, BN)};
    const int kStages = kNarrow ? ng.stages : num_stages_epi(EPI, CG, BN);
    const int kSub = kNarrow ? ng.ksub : 1;                                           // K blocks per stage
    const uint32_t kSubBytes = kNarrow ? ng.sub_bytes : stage_bytes(CG, BN);          // bytes of one K block
    const uint32_t kStageBytes = kNarrow ? ng.sub_bytes * ng.ksub : stage_bytes(CG, BN);
    const uint32_t kAOff = kNarrow ? a_box_bytes : kABytes;   // B follows the A box inside a sub-stage
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages], bar_empty[kMaxStages], bar_tfull[2], bar_tempty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t ring = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // In a pair, rank 0 is the leader: it owns the "full" and "accumulator free" barriers and issues the MMAs.
    const uint32_t cta_rank = CG == 2 ? ptx::cluster_ctarank() : 0u;
    const int first_tile = static_cast<int>(blockIdx.x) / CG;   // pairs walk the tile list together
    const int tile_stride = static_cast<int>(gridDim.x) / CG;
    const int m_tiles = (M + kBM * CG - 1) / (kBM * CG);
    const int n_tiles = (n_out + kNStep - 1) / kNStep;
    const int num_tiles = m_tiles * n_tiles;
    const int num_kb = (K + kBK - 1) / kBK;   // K blocks; a stage carries kSub of them (blocks past K read as zeros)

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_addr(&bar_full[s]), 1);
            ptx::mbar_init(ptx::smem_addr(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(ptx::smem_addr(&bar_tfull[a]), 1);
            ptx::mbar_init(ptx::smem_addr(&bar_tempty[a]), kEpiWarps * CG);   // every epilogue warp of every CTA of the group
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmA);
        ptx::prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        if constexpr (CG == 2) {
            ptx::tmem_alloc_pair(ptx::smem_addr(&tmem_base_slot), kTmemCols);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_addr(&tmem_base_slot), kTmemCols);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) ptx::cluster_sync();   // the partner's barriers exist before anything signals them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    // Programmatic dependent launch (when the host asks for it): everything above overlaps the tail of the
    // previous kernel in the stream; the roles that touch global memory wait for that kernel here. The next
    // kernel may begin its own prologue as soon as this one's CTAs start to retire.
    ptx::grid_dep_launch();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (ptx::elect_one()) {
            ptx::grid_dep_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = first_tile; ok && t < num_tiles; t += tile_stride) {
                const TileCoord tc = tile_coord(t, m_tiles, n_tiles, kNStep, kBM * CG);
                const int m0 = tc.m0 + static_cast<int>(cta_rank) * kBM;     // this CTA's rows of the tile
                const int b_row1 = kNStep == BN ? tc.n0 + BN / 2 : n_out + tc.n0;   // second half of the B rows
                for (int kb = 0; kb < num_kb; kb += kSub) {
                    if (!ptx::mbar_wait(ptx::smem_addr(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = ring + stage * kStageBytes;
                    const uint32_t sb = sa + kAOff;
                    const int k0 = kb * kBK;
                    if constexpr (CG == 1) {
                        const uint32_t full = ptx::smem_addr(&bar_full[stage]);
                        // the A box may be shorter than 128 rows; a narrow-tile stage holds kSub K blocks (blocks
                        // past K are out of range for the tensor maps: they arrive as zeros and count their bytes)
                        ptx::mbar_arrive_expect_tx(full, (a_box_bytes + kBBytes) * static_cast<uint32_t>(kSub));
                        for (int sub = 0; sub < kSub; ++sub) {
                            const uint32_t ssa = sa + sub * kSubBytes, ssb = sb + sub * kSubBytes;
                            const int kk = k0 + sub * kBK;
                            if constexpr (!A_MN) {
                                ptx::tma_load_2d(ssa, &tmA, kk, m0, full);
                            } else {
#pragma unroll
                                for (int c = 0; c < kBM / 64; ++c) ptx::tma_load_2d(ssa + c * 8192u, &tmA, m0 + 64 * c, kk, full);
                            }
                            if constexpr (!B_MN) {
                                if constexpr (kNarrow && kNStep == BN) {
                                    // plain narrow tile: its B rows are contiguous, one box of BN rows (half as many copies
                                    // to issue as two boxes of BN / 2; the copies, not the bytes, bound a skinny tile)
                                    ptx::tma_load_2d(ssb, &tmB, kk, tc.n0, full);
                                } else {
                                    ptx::tma_load_2d(ssb, &tmB, kk, tc.n0, full);
                                    ptx::tma_load_2d(ssb + kBBytes / 2, &tmB, kk, b_row1, full);
                                }
                            } else {
#pragma unroll
                                for (int c = 0; c < BN / 64; ++c) ptx::tma_load_2d(ssb + c * 8192u, &tmB, tc.n0 + 64 * c, kk, full);
                            }
                        }
                    } else {
                        // Both CTAs' bytes are counted on the LEADER's barrier: the leader announces the total,
                        // the partner only loads. (Bytes that land before the announcement leave the count
                        // negative for a moment; the phase cannot complete before the leader's arrival.)
                        const uint32_t full = ptx::map_to_cta(ptx::smem_addr(&bar_full[stage]), 0);
                        if (cta_rank == 0) ptx::mbar_arrive_expect_tx(ptx::smem_addr(&bar_full[stage]), 2 * kStageBytes);
                        if constexpr (!A_MN) {
                            ptx::tma_load_2d_pair(sa, &tmA, k0, m0, full);
                        } else {
#pragma unroll
                            for (int c = 0; c < kBM / 64; ++c) ptx::tma_load_2d_pair(sa + c * 8192u, &tmA, m0 + 64 * c, k0, full);
                        }
                        if constexpr (!B_MN) {   // this CTA's half of the B rows
                            ptx::tma_load_2d_pair(sb, &tmB, k0, cta_rank == 0 ? tc.n0 : b_row1, full);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 128; ++c)
                                ptx::tma_load_2d_pair(sb + c * 8192u, &tmB, tc.n0 + static_cast<int>(cta_rank) * (BN / 2) + 64 * c, k0, full);
                        }
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (cta_rank == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = instr_desc(std::is_same<T, __nv_bfloat16>::value ? 1u : 0u, A_MN, B_MN, CG, BN);
            constexpr uint32_t a_step = A_MN ? (2048u >> 4) : (32u >> 4);  // start-address step per K=16 slice
            constexpr uint32_t b_step = B_MN ? (2048u >> 4) : (32u >> 4);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = first_tile; ok && t < num_tiles; t += tile_stride) {
                if (!ptx::mbar_wait(ptx::smem_addr(&bar_tempty[acc]), acc_phase ^ 1u, &abort_flag)) break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kAccStride;
                for (int kb = 0; kb < num_kb; kb += kSub) {
                    if (!ptx::mbar_wait(ptx::smem_addr(&bar_full[stage]), phase, &abort_flag)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    for (int sub = 0; sub < kSub; ++sub) {
                        const uint32_t sa = ring + stage * kStageBytes + sub * kSubBytes;
                        const uint64_t da = smem_desc_sw128(sa, A_MN);
                        const uint64_t db = smem_desc_sw128(sa + kAOff, B_MN);
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k) {
                            if constexpr (CG == 2) ptx::umma_f16_pair(d_tmem, da + a_step * k, db + b_step * k, idesc, (kb | sub | k) != 0 ? 1u : 0u);
                            else ptx::umma_f16(d_tmem, da + a_step * k, db + b_step * k, idesc, (kb | sub | k) != 0 ? 1u : 0u);
                        }
                    }
                    // stage free (in both CTAs of a pair) once these MMAs retire
                    if constexpr (CG == 2) ptx::umma_commit_pair(ptx::smem_addr(&bar_empty[stage]), 3);
                    else ptx::umma_commit(ptx::smem_addr(&bar_empty[stage]));
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {   // accumulator complete (each CTA of a pair holds its own 128 rows of it)
                    if constexpr (CG == 2) ptx::umma_commit_pair(ptx::smem_addr(&bar_tfull[acc]), 3);
                    else ptx::umma_commit(ptx::smem_addr(&bar_tfull[acc]));
                }
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9) ----------------
        const int q = warp & 3;               // TMEM lane quarter this warp may read: lanes [32q, 32q+32)
        const int chunk0 = (warp - 2) >> 2;   // the two warps of a quarter take the even / the odd 32-column chunks
        ptx::grid_dep_wait();
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = first_tile; t < num_tiles; t += tile_stride) {
            const TileCoord tc = tile_coord(t, m_tiles, n_tiles, kNStep, kBM * CG);
            if (!ptx::mbar_wait(ptx::smem_addr(&bar_tfull[acc]), acc_phase, &abort_flag)) break;
            ptx::tc_fence_after_sync();
            const int row = tc.m0 + static_cast<int>(cta_rank) * kBM + q * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc) * kAccStride;
            T* crow = C + static_cast<int64_t>(row) * ldc + tc.n0;
            [[maybe_unused]] float rs = 1.0f;                 // kEpiSwiglu: this row's scale
            if constexpr (EPI == kEpiSwiglu) {
                if (row_scale != nullptr && row < M) rs = __ldg(row_scale + row);
            }
            [[maybe_unused]] uint4 gp_next[4], vp_next[4];   // kEpiDhDgv: packets requested one chunk ahead
            if constexpr (BN == kBNTiny && EPI == kEpiSwiglu) {
                // one 32-column read holds the whole accumulator: 16 gate columns, then the 16 value columns
                if (chunk0 == 0) {
                    uint32_t a[32];
                    ptx::tmem_ld_32x32(t_row, a);
                    ptx::tmem_ld_wait();
                    uint32_t out[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        out[j] = pack2<T>(silu_mul(rs * __uint_as_float(a[2 * j]), rs * __uint_as_float(a[16 + 2 * j])),
                                          silu_mul(rs * __uint_as_float(a[2 * j + 1]), rs * __uint_as_float(a[16 + 2 * j + 1])));
                    if (row < M) {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            if (tc.n0 + j * 8 < n_out)
                                *reinterpret_cast<uint4*>(crow + j * 8) = make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
                    }
                }
            }
#pragma unroll 1
            for (int c = chunk0; c < kChunks; c += kEpiWarps / 4) {
                if constexpr (EPI == kEpiSwigluBwd) {
                    uint32_t g[32], v[32];
                    ptx::tmem_ld_32x32(t_row + c * 32, g);
                    ptx::tmem_ld_32x32(t_row + BN / 2 + c * 32, v);
                    uint4 dhp[4];
                    const T* arow = aux + static_cast<int64_t>(row) * ld_aux + tc.n0 + c * 32;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool on = row < M && tc.n0 + c * 32 + j * 8 < n_out;
                        dhp[j] = on ? *reinterpret_cast<const uint4*>(arow + j * 8) : make_uint4(0, 0, 0, 0);
                    }
                    ptx::tmem_ld_wait();
                    uint32_t og[16], ov[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float dh[8];
                        unpack16<T>(dhp[j], dh);
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            float dg2[2], dv2[2];
#pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                const float gg = __uint_as_float(g[j * 8 + e + u]), vv = __uint_as_float(v[j * 8 + e + u]);
                                const float sig = sigmoid_(gg);
                                dv2[u] = dh[e + u] * (gg * sig);
                                dg2[u] = dh[e + u] * vv * (sig * (1.0f + gg * (1.0f - sig)));
                            }
                            og[j * 4 + e / 2] = pack2<T>(dg2[0], dg2[1]);
                            ov[j * 4 + e / 2] = pack2<T>(dv2[0], dv2[1]);
                        }
                    }
                    if (row < M) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int col = tc.n0 + c * 32 + j * 8;
                            if (col < n_out) {
                                *reinterpret_cast<uint4*>(crow + c * 32 + j * 8) =
                                    make_uint4(og[4 * j], og[4 * j + 1], og[4 * j + 2], og[4 * j + 3]);
                                *reinterpret_cast<uint4*>(crow + n_out + c * 32 + j * 8) =
                                    make_uint4(ov[4 * j], ov[4 * j + 1], ov[4 * j + 2], ov[4 * j + 3]);
                            }
                        }
                    }
                } else if constexpr (EPI == kEpiDhDgv) {
                    // Global traffic in a coalesced layout: instruction i of four covers rows 8i..8i+7 of this warp's
                    // 32, four lanes x 16 B = the chunk's 64 contiguous bytes of a row (whole sectors; a quarter of
                    // the cache lines per instruction that one-row-per-lane accesses touch). The accumulator is
                    // row-per-lane, so packets change layout through the warp's staging buffer.
                    // The stored gate / value packets of the NEXT chunk are requested while this chunk is worked
                    // on, so their latency (L2 or HBM) overlaps the arithmetic instead of heading it.
                    constexpr int kStride = kEpiWarps / 4;
                    const int cr = lane >> 2, cp = lane & 3;
                    const int row0 = tc.m0 + static_cast<int>(cta_rank) * kBM + q * 32;
                    const uint32_t sbuf = ring + static_cast<uint32_t>(kStages) * kStageBytes + static_cast<uint32_t>(warp - 2) * kEpiStageBytes;
                    // rows cr + 8 i share (row >> 1) & 3 with row cr, so one swizzled address serves all four i
                    const uint32_t s_co = sbuf + static_cast<uint32_t>(cr) * kEpiRowPitch + ((static_cast<uint32_t>(cp) ^ ((static_cast<uint32_t>(cr) >> 1) & 3u)) << 4);   // + i * 8 rows
                    const uint32_t s_row = sbuf + static_cast<uint32_t>(lane) * kEpiRowPitch;   // piece j at + ((j ^ sw_row) << 4)
                    const uint32_t sw_row = (static_cast<uint32_t>(lane) >> 1) & 3u;
                    uint32_t a[32];
                    ptx::tmem_ld_32x32(t_row + c * 32, a);
                    auto fetch = [&](int cc) {
                        const int col = tc.n0 + cc * 32 + cp * 8;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = row0 + i * 8 + cr;
                            const bool on = rr < M && col < n_out;
                            const T* gptr = aux + static_cast<int64_t>(rr) * ld_aux + col;
                            gp_next[i] = on ? ld_stream16(reinterpret_cast<const uint4*>(gptr)) : make_uint4(0, 0, 0, 0);
                            vp_next[i] = on ? ld_stream16(reinterpret_cast<const uint4*>(gptr + n_out)) : make_uint4(0, 0, 0, 0);
                        }
                    };
                    if (c == chunk0) fetch(c);
                    uint4 gp[4], vp[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) ptx::sts128(s_co + static_cast<uint32_t>(i) * 8u * kEpiRowPitch, gp_next[i]);
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) gp[j] = ptx::lds128(s_row + ((static_cast<uint32_t>(j) ^ sw_row) << 4));
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i) ptx::sts128(s_co + static_cast<uint32_t>(i) * 8u * kEpiRowPitch, vp_next[i]);
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) vp[j] = ptx::lds128(s_row + ((static_cast<uint32_t>(j) ^ sw_row) << 4));
                    __syncwarp();
                    if (c + kStride < kNStep / 32) fetch(c + kStride);
                    ptx::tmem_ld_wait();
                    uint4 og[4], ov[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float gg[8], vv[8], dg[8], dv[8];
                        unpack16<T>(gp[j], gg);
                        unpack16<T>(vp[j], vv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float dh = __uint_as_float(a[j * 8 + e]);
                            const float sig = sigmoid_(gg[e]);
                            dv[e] = dh * (gg[e] * sig);
                            dg[e] = dh * vv[e] * (sig * (1.0f + gg[e] * (1.0f - sig)));
                        }
                        og[j] = pack16<T>(dg);
                        ov[j] = pack16<T>(dv);
                    }
                    // read once / written once: streaming stores keep the GEMM operands in L2
                    const int ocol = tc.n0 + c * 32 + cp * 8;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) ptx::sts128(s_row + ((static_cast<uint32_t>(j) ^ sw_row) << 4), half == 0 ? og[j] : ov[j]);
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = row0 + i * 8 + cr;
                            const uint4 v = ptx::lds128(s_co + static_cast<uint32_t>(i) * 8u * kEpiRowPitch);
                            if (rr < M && ocol < n_out)
                                st_stream16(reinterpret_cast<uint4*>(C + static_cast<int64_t>(rr) * ldc + ocol + (half == 0 ? 0 : n_out)), v);
                        }
                        __syncwarp();
                    }
                } else {
                    uint32_t out[16];
                    if constexpr (EPI == kEpiSwiglu || EPI == kEpiSwigluSave) {
                        uint32_t g[32], v[32];
                        ptx::tmem_ld_32x32(t_row + c * 32, g);
                        ptx::tmem_ld_32x32(t_row + BN / 2 + c * 32, v);
                        ptx::tmem_ld_wait();
                        if constexpr (EPI == kEpiSwiglu) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                out[j] = pack2<T>(silu_mul(rs * __uint_as_float(g[2 * j]), rs * __uint_as_float(v[2 * j])),
                                                  silu_mul(rs * __uint_as_float(g[2 * j + 1]), rs * __uint_as_float(v[2 * j + 1])));
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                out[j] = pack2<T>(silu_mul(__uint_as_float(g[2 * j]), __uint_as_float(v[2 * j])),
                                                  silu_mul(__uint_as_float(g[2 * j + 1]), __uint_as_float(v[2 * j + 1])));
                        }
                        if constexpr (EPI == kEpiSwigluSave) {
                            if (row < M) {
                                T* prow = C2 + static_cast<int64_t>(row) * ld_aux + tc.n0 + c * 32;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    if (tc.n0 + c * 32 + j * 8 < n_out) {
                                        uint32_t pg[4], pv[4];
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            pg[e] = pack2<T>(__uint_as_float(g[j * 8 + 2 * e]), __uint_as_float(g[j * 8 + 2 * e + 1]));
                                            pv[e] = pack2<T>(__uint_as_float(v[j * 8 + 2 * e]), __uint_as_float(v[j * 8 + 2 * e + 1]));
                                        }
                                        st_stream16(reinterpret_cast<uint4*>(prow + j * 8), make_uint4(pg[0], pg[1], pg[2], pg[3]));
                                        st_stream16(reinterpret_cast<uint4*>(prow + n_out + j * 8), make_uint4(pv[0], pv[1], pv[2], pv[3]));
                                    }
                                }
                            }
                        }
                    } else {
                        uint32_t a[32];
                        ptx::tmem_ld_32x32(t_row + c * 32, a);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) out[j] = pack2<T>(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]));
                    }
                    if (row < M) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int col = tc.n0 + c * 32 + j * 8;
                            // n_out is a multiple of 8: a 16-byte vector is entirely in or out; a 48-column tile ends
                            // in the middle of its second chunk
                            if (col < n_out && (kNStep % 32 == 0 || c * 32 + j * 8 < kNStep))
                                *reinterpret_cast<uint4*>(crow + c * 32 + j * 8) =
                                    make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
                        }
                    }
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {   // the accumulator is free when every epilogue warp (of both CTAs of a pair) has drained it
                if (CG == 2 && cta_rank != 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_addr(&bar_tempty[acc]), 0));
                else ptx::mbar_arrive(ptx::smem_addr(&bar_tempty[acc]));
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    // A pair leaves together: the leader's MMAs read the partner's shared memory and the partner signals
    // barriers in the leader's, so neither may exit (or free tensor memory) before both are done.
    if constexpr (CG == 2) ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if constexpr (CG == 2) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
        else ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && abort_flag != 0) atomicExch(status, MGR_ERR_DEVICE_TIMEOUT);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup: the library does not link
// libcuda, so it still loads (for its host-side checks) on a machine without a driver.
EncodeTiledFn encode_tiled_fn() {
    static std::atomic<EncodeTiledFn> fn{nullptr};
    if (fn.load(std::memory_order_relaxed) == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        fn.store(reinterpret_cast<EncodeTiledFn>(p), std::memory_order_relaxed);
    }
    return fn.load(std::memory_order_relaxed);
}

// Tensor map over a row-major [outer, inner] matrix of 16-bit elements with leading dimension ld
// (elements): box = 64 (inner) x box_outer, 128-byte swizzle, out-of-range elements read as zero.
// K-major operands pass (inner = K, outer = rows, box_outer = 128); MN-major operands are stored
// [K, rows] and pass (inner = rows, outer = K, box_outer = 64).
bool make_tmap(CUtensorMap* tm, const void* base, int64_t outer, int64_t inner, int64_t ld, uint32_t box_outer, int dtype) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {64, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = dtype == MGR_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* gemm_status_ptr(const DeviceInfo& di) {
    static std::atomic<int*> cache[kMaxDevices];   // racing first calls store the same address
    if (cache[di.device].load(std::memory_order_relaxed) == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_gemm_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cache[di.device].store(static_cast<int*>(p), std::memory_order_relaxed);
    }
    return cache[di.device].load(std::memory_order_relaxed);
}

struct GemmArgs {
    void* c2;   // second output (kEpiSwigluSave: the stored projection), else nullptr
    void* c;
    const void* a;
    const void* b;
    const void* aux;
    int64_t m, n_out, k;       // problem: C tile grid covers m x n_out, contraction length k
    int64_t b_rows;            // logical rows of B (n_out, or 2 n_out for the gate|value split)
    int64_t lda, ldb, ldc, ld_aux;
    int dtype;
    const float* row_scale = nullptr;   // kEpiSwiglu only
};

// SMs the GEMM kernels may occupy (0 = all). A caller that overlaps a collective with a GEMM lowers it so
// that the communication kernel finds free SMs next to the persistent GEMM CTAs.
std::atomic<int> g_sm_limit{0};

// MGR_GEMM_CTA_GROUP=1|2 pins the single-CTA or the CTA-pair kernels; unset = automatic.
int forced_cta_group() { return overrides().cta_group; }

// GEMM kernels are launched with programmatic stream serialization: the prologue (barriers, tensor memory,
// descriptor prefetch) of a GEMM overlaps the tail of the kernel before it in the stream (1-2.5 us per launch in a
// chain of short GEMMs). Not while an SM limit is set: the early CTAs of the next GEMM would park on the SMs that
// the limit keeps free for a collective. MGR_GEMM_PDL=0 switches it off.
bool pdl_enabled() {
    return overrides().pdl != 0 && g_sm_limit.load(std::memory_order_relaxed) == 0;
}

template <int EPI, bool A_MN, bool B_MN, int CG, typename T, int BN = kBN>
int launch_gemm(const GemmArgs& g, const DeviceInfo& di, cudaStream_t s) {
    static std::atomic<bool> attr[kMaxDevices];
    constexpr uint32_t kGemmSmem = gemm_smem_epi(EPI, CG, BN);
    if (!attr[di.device].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(gemm_kernel<EPI, A_MN, B_MN, CG, T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kGemmSmem)) != cudaSuccess) {
            (void)cudaGetLastError();
            return MGR_ERR_CUDA;
        }
        attr[di.device].store(true, std::memory_order_release);
    }
    CUtensorMap tmA, tmB;
    // A problem of fewer than 128 rows brings in only the rows it has (rounded up to 8): the rest of the
    // 128-row operand tile stays whatever shared memory held, which only reaches output rows >= M, and those
    // are never stored. At 16 rows this cuts the bytes per K step from 24 KB to 10 KB (narrow tiles).
    const uint32_t a_rows = (CG == 1 && !A_MN && g.m < kBM) ? static_cast<uint32_t>((g.m + 7) / 8 * 8) : static_cast<uint32_t>(kBM);
    const uint32_t a_box_bytes = A_MN ? kABytes : a_rows * kBK * 2;
    const bool okA = A_MN ? make_tmap(&tmA, g.a, g.k, g.m, g.lda, 64, g.dtype) : make_tmap(&tmA, g.a, g.m, g.k, g.lda, a_rows, g.dtype);
    // K-major B: a single CTA loads its B rows as two boxes of BN/2 rows (second one at the value rows for the
    // gate|value split); a pair loads one box of 128 rows per CTA.
    const bool okB = B_MN ? make_tmap(&tmB, g.b, g.k, g.b_rows, g.ldb, 64, g.dtype)
                          : make_tmap(&tmB, g.b, g.b_rows, g.k, g.ldb, CG == 2 ? 128 : ((BN < kBN && n_step_of(EPI, BN) == BN) ? BN : BN / 2), g.dtype);
    if (!okA || !okB) return MGR_ERR_CUDA;
    int* status = gemm_status_ptr(di);
    if (status == nullptr) return MGR_ERR_CUDA;
    constexpr int n_step = n_step_of(EPI, BN);
    const int64_t tiles = ((g.m + kBM * CG - 1) / (kBM * CG)) * ((g.n_out + n_step - 1) / n_step);
    const int limit = g_sm_limit.load(std::memory_order_relaxed);
    const int sms = (limit > 0 && limit < di.sm_count) ? limit : di.sm_count;
    const int64_t slots = sms / CG > 0 ? sms / CG : 1;   // CTAs (pairs) that can be resident at once
    const unsigned grid = static_cast<unsigned>((tiles < slots ? tiles : slots) * CG);
    T* c = static_cast<T*>(g.c);
    T* c2 = static_cast<T*>(g.c2);
    const T* aux = static_cast<const T*>(g.aux);
    const int m = static_cast<int>(g.m), n_out = static_cast<int>(g.n_out), k = static_cast<int>(g.k);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = kGemmSmem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    unsigned na = 0;
    if constexpr (CG == 2) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = 2;
        at[na].val.clusterDim.y = 1;
        at[na].val.clusterDim.z = 1;
        ++na;
    }
    if (pdl_enabled()) {   // the kernel's prologue may overlap the tail of the previous kernel in the stream
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = at;
    cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, gemm_kernel<EPI, A_MN, B_MN, CG, T, BN>, tmA, tmB, c, c2, aux, m, n_out, k, g.ldc, g.ld_aux,
                           a_box_bytes, g.row_scale, status) != cudaSuccess) {
        (void)cudaGetLastError();
        return MGR_ERR_LAUNCH_FAILED;
    }
    return launch_status();
}

// Choice between the single-CTA and the CTA-pair kernels, from measurements on B200 (1 kW power cap):
//   * in cycles the pair kernels are clearly better: tensor pipe active 90-94 % against 77-79 % at 4096^3,
//     15 % fewer cycles (deeper ring, half the B traffic per CTA);
//   * a short burst of GEMMs (config 4: 0.2-0.4 ms each) runs near the maximum clock and gains from that:
//     1.21 against 1.15 PFLOP/s for the whole MLP step;
//   * a long run of large GEMMs (config 5 on one GPU: 5-10 ms each) is held at the power cap, where the pair
//     kernels settle at about 1.0 GHz against 1.25 GHz for the single-CTA ones and lose 4 %
//     (1.19 against 1.24 PFLOP/s).
// Hence: pairs for GEMMs below 2 TFLOP of work, single CTAs above. MGR_GEMM_CTA_GROUP overrides.
constexpr double kPairFlopLimit = 2.0e12;

template <int EPI, bool A_MN, bool B_MN, typename T>
int launch_gemm_cg(const GemmArgs& g, const DeviceInfo& di, cudaStream_t s) {
    // Few tiles (a skinny M, as in decoding): the 256-column tiles would leave most SMs without work while a
    // handful stream the whole weight matrix; 64-column tiles spread it over 4x as many CTAs.
    if constexpr ((EPI == kEpiPlain || EPI == kEpiSwiglu) && !A_MN && !B_MN) {
        constexpr int wide_step = n_step_of(EPI, kBN);
        constexpr int small_step = n_step_of(EPI, kBNSmall);
        const int64_t m_tiles = (g.m + kBM - 1) / kBM;
        const int64_t wide_tiles = m_tiles * ((g.n_out + wide_step - 1) / wide_step);
        const int64_t small_tiles = m_tiles * ((g.n_out + small_step - 1) / small_step);
        // MGR_GEMM_NARROW = 0: never; 1 (or 64): 64-column tiles; 32: 32-column tiles; unset: automatic.
        // Measured on B200 (fp16, D 4096, F 6912, CUDA graphs): the w3 GEMM of a 16-row batch has 16 / 64 / 128
        // tiles at 256 / 64 / 32 columns and takes 32 / 18 / 16 us; the fused projection (54 / 216 / 432 tiles)
        // 36 / 26 / 27 us. So: 32 columns only while 64 would still leave half the SMs idle.
        const int pinned = overrides().narrow;
        int bn = 0;
        if (pinned >= 0) {
            bn = pinned == 0 ? 0 : (pinned == 32 ? kBNTiny : (pinned == 96 && EPI == kEpiSwiglu ? kBNMid : kBNSmall));
        } else if (wide_tiles * 2 <= di.sm_count && m_tiles <= 3) {
            // Up to 384 rows only: from 4 row tiles on, every narrow tile re-reads its 128 rows of A and the wide
            // tiling wins again (w3 GEMM at 512 rows: 37.9 us wide against 42.3 us narrow; at 256 rows 36.6 against 21.8).
            // Among the narrow widths: the one with the least (rounds over the SMs) x (tile width + a fixed cost per
            // tile of about 16 columns' worth). For the 16-row batch above that is 32 columns for w3 (128 tiles, one
            // round) and 48 + 48 for the projection (144 tiles, one round, where 32 + 32 needs two and 16 + 16 three).
            (void)small_tiles;
            const int widths[3] = {kBNTiny, kBNSmall, kBNMid};
            int64_t best = 0;
            for (int i = 0; i < (EPI == kEpiSwiglu ? 3 : 2); ++i) {
                const int step = widths[i] / (EPI == kEpiSwiglu ? 2 : 1);
                const int64_t tiles = m_tiles * ((g.n_out + step - 1) / step);
                const int64_t rounds = (tiles + di.sm_count - 1) / di.sm_count;
                const int64_t cost = rounds * (widths[i] + 16);
                if (bn == 0 || cost < best) bn = widths[i], best = cost;
            }
        }
        if (bn == kBNTiny) return launch_gemm<EPI, A_MN, B_MN, 1, T, kBNTiny>(g, di, s);
        if (bn == kBNSmall) return launch_gemm<EPI, A_MN, B_MN, 1, T, kBNSmall>(g, di, s);
        if constexpr (EPI == kEpiSwiglu) {
            if (bn == kBNMid) return launch_gemm<EPI, A_MN, B_MN, 1, T, kBNMid>(g, di, s);
        }
    }
    int cg = forced_cta_group();
    if (cg == 0) {
        const double flops = 2.0 * static_cast<double>(g.m) * static_cast<double>(g.b_rows) * static_cast<double>(g.k);
        cg = flops < kPairFlopLimit ? 2 : 1;
    }
    if (cg == 2 && di.sm_count % 2 == 0) {
        const int st = launch_gemm<EPI, A_MN, B_MN, 2, T>(g, di, s);
        if (st != MGR_ERR_LAUNCH_FAILED) return st;
        // a cluster of two could not be placed (e.g. a partitioned device): the single-CTA kernels need none
    }
    return launch_gemm<EPI, A_MN, B_MN, 1, T>(g, di, s);
}

template <int EPI, bool A_MN, bool B_MN>
int launch_gemm_dtype(const GemmArgs& g, const DeviceInfo& di, cudaStream_t s) {
    if (g.dtype == MGR_F16) return launch_gemm_cg<EPI, A_MN, B_MN, __half>(g, di, s);
    return launch_gemm_cg<EPI, A_MN, B_MN, __nv_bfloat16>(g, di, s);
}

int gemm_check(int64_t m, int64_t n, int64_t k, int dtype) {
    if (dtype != MGR_F16 && dtype != MGR_BF16) return MGR_ERR_BAD_DTYPE;
    if (m < 0 || n < 1 || k < 1) return MGR_ERR_BAD_SHAPE;
    if (n % 8 != 0 || k % 8 != 0) return MGR_ERR_BAD_SHAPE;  // 16-byte rows for TMA and for the vector stores
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return MGR_ERR_TOO_LARGE;
    return MGR_OK;
}

}  // namespace

int gemm_status_fetch(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        return MGR_ERR_CUDA;
    }
    if (clear && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)) != cudaSuccess) (void)cudaGetLastError();
    }
    return v;
}

int gemm_status_poke(int value) {
    return cudaMemcpyToSymbol(g_gemm_status, &value, sizeof(int)) == cudaSuccess ? MGR_OK : ((void)cudaGetLastError(), MGR_ERR_CUDA);
}

}  // namespace mgr

using namespace mgr;

// Leading dimension of an operand with `rows` logical rows and contraction length k.
static int check_ld(int64_t ld, int64_t rows, int64_t k, int mn_major) {
    const int64_t need = mn_major ? rows : k;
    return ld >= need && ld % 8 == 0;
}

extern "C" int mgr_gemm(void* c, const void* a, const void* b, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                        int64_t ldc, int a_mn_major, int b_mn_major, int dtype, void* stream) {
    int st = gemm_check(m, n, k, dtype);
    if (st != MGR_OK) return st;
    if (m % 8 != 0 && a_mn_major) return MGR_ERR_BAD_SHAPE;  // rows of an MN-major A are its inner dimension
    if (!check_ld(lda, m, k, a_mn_major) || !check_ld(ldb, n, k, b_mn_major) || ldc < n || ldc % 8 != 0) return MGR_ERR_BAD_SHAPE;
    if (m == 0) return MGR_OK;
    if (c == nullptr || a == nullptr || b == nullptr) return MGR_ERR_NULL_PTR;
    if (!aligned_to(c, 16) || !aligned_to(a, 16) || !aligned_to(b, 16)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const GemmArgs g{nullptr, c, a, b, nullptr, m, n, k, n, lda, ldb, ldc, 0, dtype};
    if (!a_mn_major && !b_mn_major) return launch_gemm_dtype<kEpiPlain, false, false>(g, di, s);
    if (!a_mn_major && b_mn_major) return launch_gemm_dtype<kEpiPlain, false, true>(g, di, s);
    if (a_mn_major && !b_mn_major) return launch_gemm_dtype<kEpiPlain, true, false>(g, di, s);
    return launch_gemm_dtype<kEpiPlain, true, true>(g, di, s);
}

extern "C" int mgr_gemm_tn(void* c, const void* a, const void* b, int64_t m, int64_t n, int64_t k, int64_t lda,
                           int64_t ldb, int64_t ldc, int dtype, void* stream) {
    return mgr_gemm(c, a, b, m, n, k, lda, ldb, ldc, 0, 0, dtype, stream);
}

extern "C" int mgr_swiglu_fused_fwd_scaled(void* h, const void* x, const void* w12, const float* row_scale, int64_t m, int64_t d,
                                           int64_t f, int dtype, void* stream) {
    int st = gemm_check(m, f, d, dtype);
    if (st != MGR_OK) return st;
    if (m == 0) return MGR_OK;
    if (h == nullptr || x == nullptr || w12 == nullptr) return MGR_ERR_NULL_PTR;
    if (!aligned_to(h, 16) || !aligned_to(x, 16) || !aligned_to(w12, 16) || !aligned_to(row_scale, 4)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    GemmArgs g{nullptr, h, x, w12, nullptr, m, f, d, 2 * f, d, d, f, 0, dtype};
    g.row_scale = row_scale;
    return launch_gemm_dtype<kEpiSwiglu, false, false>(g, di, static_cast<cudaStream_t>(stream));
}

extern "C" int mgr_swiglu_fused_fwd(void* h, const void* x, const void* w12, int64_t m, int64_t d, int64_t f, int dtype,
                                    void* stream) {
    return mgr_swiglu_fused_fwd_scaled(h, x, w12, nullptr, m, d, f, dtype, stream);
}

extern "C" int mgr_swiglu_fused_bwd(void* dgv, const void* dh, const void* x, const void* w12, int64_t m, int64_t d,
                                    int64_t f, int dtype, void* stream) {
    int st = gemm_check(m, f, d, dtype);
    if (st != MGR_OK) return st;
    if (m == 0) return MGR_OK;
    if (dgv == nullptr || dh == nullptr || x == nullptr || w12 == nullptr) return MGR_ERR_NULL_PTR;
    if (!aligned_to(dgv, 16) || !aligned_to(dh, 16) || !aligned_to(x, 16) || !aligned_to(w12, 16)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    const GemmArgs g{nullptr, dgv, x, w12, dh, m, f, d, 2 * f, d, d, 2 * f, f, dtype};
    return launch_gemm_dtype<kEpiSwigluBwd, false, false>(g, di, static_cast<cudaStream_t>(stream));
}

extern "C" int mgr_swiglu_fused_fwd_save(void* h, void* gv, const void* x, const void* w12, int64_t m, int64_t d, int64_t f,
                                         int dtype, void* stream) {
    int st = gemm_check(m, f, d, dtype);
    if (st != MGR_OK) return st;
    if (m == 0) return MGR_OK;
    if (h == nullptr || gv == nullptr || x == nullptr || w12 == nullptr) return MGR_ERR_NULL_PTR;
    if (!aligned_to(h, 16) || !aligned_to(gv, 16) || !aligned_to(x, 16) || !aligned_to(w12, 16)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    const GemmArgs g{gv, h, x, w12, nullptr, m, f, d, 2 * f, d, d, f, 2 * f, dtype};
    return launch_gemm_dtype<kEpiSwigluSave, false, false>(g, di, static_cast<cudaStream_t>(stream));
}

extern "C" int mgr_swiglu_dh_dgv(void* dgv, const void* dy, const void* w3, const void* gv, int64_t m, int64_t d, int64_t f,
                                 int dtype, void* stream) {
    int st = gemm_check(m, f, d, dtype);
    if (st != MGR_OK) return st;
    if (m == 0) return MGR_OK;
    if (dgv == nullptr || dy == nullptr || w3 == nullptr || gv == nullptr) return MGR_ERR_NULL_PTR;
    if (!aligned_to(dgv, 16) || !aligned_to(dy, 16) || !aligned_to(w3, 16) || !aligned_to(gv, 16)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    // dh[m, f] = dy[m, d] w3[d, f]: A K-major (pitch d), B MN-major (stored [k = d, n = f], pitch f)
    const GemmArgs g{nullptr, dgv, dy, w3, gv, m, f, d, f, d, f, 2 * f, 2 * f, dtype};
    return launch_gemm_dtype<kEpiDhDgv, false, true>(g, di, static_cast<cudaStream_t>(stream));
}

extern "C" int mgr_gemm_set_sm_limit(int sms) {
    if (sms < 0) sms = 0;
    return g_sm_limit.exchange(sms, std::memory_order_relaxed);
}
