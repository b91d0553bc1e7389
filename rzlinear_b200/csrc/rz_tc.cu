// Tensor-core (tcgen05 + TMEM + TMA) kernels of the RzLinear path for sm_100a.
//
// One persistent, warp-specialised kernel template covers the three contractions:
//   OP_FWD  Y [M,N] = X  [M,K] . W[K,N]      A = X tile  (K-major),  B = W slice (N-major)
//   OP_DX   dX[M,K] = dY [M,N] . W[K,N]^T    A = dY tile (K-major),  B = W slice (K-major)
//   OP_DW   dH     += dY^T[N,M] . X[M,K]     A = dY tile (M-major),  B = X tile  (N-major): the TRANSPOSE of the
//                                             weight-gradient block, so that a warp's 32 accumulator rows are 32
//                                             consecutive words of a slice row and reductions need no transpose
// CTAS = 1, RB = 1: a CTA owns a 128 x 256 output block (tcgen05.mma cta_group::1, M = 128).
// CTAS = 2, RB = 1: two CTAs of a cluster own a 256 x 256 block (cta_group::2, M = 256): each CTA
//           stages its 128 rows of A and its 128 columns of B.  The leader CTA (rank 0) issues the
//           MMAs for both; the barriers that gate them live in the leader.
// CTAS = 2, RB = 2: the pair owns a 512 x 256 block as two M = 256 MMAs per K-step that share B: each CTA
//           stages 2 x 128 rows of A and 128 columns of B, i.e. 48 KB per 1024 tensor-clocks instead of
//           32 KB per 512.  The main loop is bound by operand bytes per flop moved through an SM (L2 -> SM
//           reads of about 50 B/clk, and the shared-memory port that TMA writes and the MMAs' operand reads
//           share), so this is the fast configuration; it is used whenever the output has at least 512 rows.
// SPLIT = 1 (fp32 precision on the tensor cores, RB = 1 only): operands are fp32; four extra warps split every
//           staged tile in shared memory into hi = the tf32-representable part and lo = x - hi, and each K-step
//           issues hi*hi + hi*lo + lo*hi (three tf32 MMAs, fp32 accumulate): fp32-grade results (the dropped
//           lo*lo term and the rounding of lo are of relative order 2^-22) at a third of the tf32 rate.
// Accumulators live in TMEM (512 columns): with RB = 1 two 256-column buffers alternate so the epilogue of
// one block overlaps the main loop of the next; with RB = 2 both halves are accumulators of one block.
// Warp 0 produces (TMA loads into a ring of 128-byte-swizzled shared-memory tiles), warp 1 issues
// tcgen05.mma, 4*RB epilogue warps drain TMEM: they scale/bias/convert and store (FWD, DX) or scatter-add
// into the hashed gradient with warp-wide coalesced reductions (DW).  EW = 4 (DW, RB = 1): sixteen epilogue
// warps for weight gradients of short contractions, whose scatter outlasts the main loop.
//
// The virtual weight is never materialised.  For every pipeline stage the producer warp computes
// the hash-tile offsets in registers and TMA-loads the matching rows of the slice.  TMA needs a
// 16-byte aligned start, and a slice starts at any element, so FWD and DX read a "shadow" of the
// hashed array: NS element-shifted copies in the compute type (NS = 8 bf16 / 4 tf32); the copy
// whose shift equals offset mod NS holds the slice at an aligned position.  (Twice as many copies would
// align rows to 32-byte sectors - four L2 sectors per 128-byte row instead of five, worth 8 % when emulated -
// but the larger footprint costs more L2 misses than that; measured, not adopted.)  The shadow tensor map
// is 3-D {element, slice row (stride BN), copy}.
//
// Every TMA load is a plain per-CTA copy of this GPU's memory; no kernel touches peer-GPU memory.
// Every mbarrier wait is bounded: a wait that runs out records a code in the device status word and
// all roles leave their loops, the producer waits for its loads in flight, the MMA thread for its
// MMAs, TMEM is freed and the kernel returns.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "rz_common.h"
#include "rz_ptx.cuh"

using namespace rzptx;

namespace {

constexpr int OP_FWD = 0, OP_DX = 1, OP_DW = 2;

constexpr int TILE_R = 128;  // rows per CTA and accumulator (MMA M = 128 * CTAS)
constexpr int A_BLOCK_BYTES = 16384;  // one 128-row block of A per stage
constexpr int BATCH = 8;     // pipeline stages per hash batch of the producer warp
constexpr int MAX_TPS = 8;   // B boxes per stage at most
constexpr int GROUP_ROWS = 8;   // row tiles per rasterisation group (4 when a tile has two row blocks)

// Shared-memory budget (227 KB per CTA): the operand ring takes what the other parts leave.
// The weight-gradient epilogue reduces straight from registers and needs no staging, so its ring gets the space.
constexpr int SMEM_TABLE = 3 * BATCH * MAX_TPS * 4;
constexpr int MAX_STAGES = 7;
constexpr int SMEM_BARS = (3 * MAX_STAGES + 5) * 8;
constexpr int SMEM_LIMIT = 232448;
// per epilogue warp: a 32-row x 128-byte store staging tile (FWD, DX); nothing for the weight gradient
// `ew`: epilogue warps per TMEM lane quarter and row block (weight gradient of short contractions: 4)
__host__ __device__ constexpr int smem_epi(int op, int rb, int ew = 1) { return op == OP_DW ? 0 : 4 * rb * ew * 4096; }
__host__ __device__ constexpr int load_bytes(int ctas, int rb, int nc) { return rb * A_BLOCK_BYTES + (nc / ctas) * 128; }
__host__ __device__ constexpr int stage_bytes(int ctas, int rb, int split, int nc) { return load_bytes(ctas, rb, nc) * (split ? 2 : 1); }
__host__ __device__ constexpr int num_stages(int op, int ctas, int rb, int split, int nc, int ew = 1)
{
    int n = (SMEM_LIMIT - 1024 - 16 - SMEM_BARS - SMEM_TABLE - smem_epi(op, rb, ew)) / stage_bytes(ctas, rb, split, nc);
    return n > MAX_STAGES ? MAX_STAGES : n;
}
__host__ __device__ constexpr int smem_total(int op, int ctas, int rb, int split, int nc, int ew = 1)
{
    return num_stages(op, ctas, rb, split, nc, ew) * stage_bytes(ctas, rb, split, nc) + smem_epi(op, rb, ew) + SMEM_TABLE + SMEM_BARS +
           16 + 1024;
}
__host__ __device__ constexpr int num_threads(int rb, int split, int ew = 1) { return 64 + 128 * rb * ew + (split ? 128 : 0); }

struct TcParams {
    RzHash hash;
    uint32_t M, K, N;
    uint32_t rows, cols;        // output extents (elements)
    uint32_t tiles_r, tiles_c;
    uint32_t nchunks;           // pipeline stages along the whole contraction
    uint32_t nsplit, chunks_per_split;   // blocks from index n_main on are split into nsplit parts of the contraction
    uint32_t n_main;                      // blocks [0, n_main) run their whole contraction in one work item
    uint32_t total_items;
    uint32_t units;             // > 0: the launch's (block, stage) units are dealt out in equal ranges (tiles * nchunks)
    uint32_t br;                // slice rows per B box (FWD: min(BK, stage depth); DX: min(BK, B columns of this CTA))
    uint32_t kparts;            // FWD: B boxes along the contraction per 128-byte column block (stage depth / br)
    uint32_t group_rows;        // row tiles per rasterisation group
    uint32_t a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep;  // descriptor strides, bytes
    uint32_t a_layout, b_layout;                            // descriptor swizzle layout type
    uint32_t idesc;
    float alpha;
    int relu;
    const float *bias;
    void *out;
    float *dH;
    float *ws;                  // FWD / DX with a split contraction: fp32 partial sums [rows][cols]
    WaitCtx wait;               // where bounded waits report
    uint32_t tma_store;         // FWD / DX: write the output with bulk tensor stores (0 = plain 16-byte stores)
};

__device__ __forceinline__ void wait_cycles(uint32_t bar, uint32_t parity, long long cycles)
{
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > cycles) break;
}

template <int OP, bool TF32, int CTAS, int RB, int SPLIT, int NC, int EW>
__global__ void __launch_bounds__(num_threads(RB, SPLIT, EW), 1)
rz_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
             const __grid_constant__ CUtensorMap mapC, const TcParams p)
{
    constexpr int ES = TF32 ? 4 : 2;        // operand element size
    constexpr int EPR = 128 / ES;           // elements per 128-byte swizzle row
    constexpr int KC = EPR;                 // contraction elements per stage
    constexpr int NS = 16 / ES;             // shifted shadow copies
    constexpr int MMAS = 4;                 // tcgen05.mma per stage (K = 16 bf16 / 8 tf32 each)
    constexpr int ATOM = KC * 128;          // bytes of one 128-byte-wide column block of an MN-major tile
    constexpr int TILE_C = NC;              // columns of the block (MMA N)
    constexpr int B_COLS = TILE_C / CTAS;   // columns of B this CTA stages
    constexpr int B_BYTES = B_COLS * 128;
    constexpr int A_BYTES = RB * A_BLOCK_BYTES;
    constexpr int LOAD_BYTES = A_BYTES + B_BYTES;                 // what TMA brings per stage and CTA
    constexpr int STAGE_BYTES = LOAD_BYTES * (SPLIT ? 2 : 1);     // SPLIT: the lo parts sit LOAD_BYTES above the hi parts
    constexpr int STAGES = num_stages(OP, CTAS, RB, SPLIT, NC, EW);
    constexpr bool PAIR_LOADS = (CTAS == 2) && !SPLIT;            // loads of both CTAs counted on the leader's barrier
    constexpr int EPI_WARPS = 4 * RB * EW;
    static_assert(EW == 1 || (OP == OP_DW && !SPLIT && ((RB == 1 && EW == 4) || (RB == 2 && EW == 2))),
                  "extra epilogue warps: weight gradient only (sixteen warps either way)");
    static_assert(!SPLIT || (TF32 && RB == 1), "split precision: fp32 operands, one row block");
    constexpr int SMEM_RING = STAGES * STAGE_BYTES;
    constexpr int SMEM_EPI_OP = smem_epi(OP, RB, EW);
    // accumulator sets in TMEM: 2 = double-buffered; 1 when both halves are in use by one block (two row blocks, or
    // the main + correction accumulators of split precision)
    constexpr int NBUF = (RB == 2 || SPLIT) ? 1 : 2;
    static_assert(STAGE_BYTES == stage_bytes(CTAS, RB, SPLIT, NC), "stage size");
    static_assert(NC == 256 || (CTAS == 1 && RB == 1), "narrow blocks: single CTA only");
    static_assert(2 * RB * NC <= 512 || RB == 2, "TMEM columns");
    // Split precision keeps the hi*hi sums and the (2^-11 smaller) hi*lo + lo*hi corrections in separate accumulators:
    // the tensor core truncates when it adds into an fp32 accumulator (about 2e-8 of the accumulator per MMA), so
    // the corrections must not cost the main chain two more truncating adds per K-step.  Chains are further bounded
    // by splitting long contractions on the host side.
    constexpr int CORR_COL = NC;            // TMEM column offset of the correction accumulator (SPLIT only)
    static_assert(RB == 1 || CTAS == 2, "two row blocks only with CTA pairs");
    constexpr int A_ATOMS = TILE_R / EPR;
    constexpr int B_ATOMS = B_COLS / EPR;
    constexpr int PAIR_R = TILE_R * CTAS;   // rows of one accumulator across the pair
    constexpr int ITEM_R = PAIR_R * RB;     // rows of a work item
    static_assert(STAGES <= MAX_STAGES, "barrier storage");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    float *epi_scratch = reinterpret_cast<float *>(smem_gen + SMEM_RING);
    uint32_t *tab_x = reinterpret_cast<uint32_t *>(smem_gen + SMEM_RING + SMEM_EPI_OP);
    uint32_t *tab_y = tab_x + BATCH * MAX_TPS;
    uint32_t *tab_z = tab_y + BATCH * MAX_TPS;
    const uint32_t bars = smem_base + SMEM_RING + SMEM_EPI_OP + SMEM_TABLE;
    const uint32_t bar_full = bars;                           // [STAGES]  used in the leader CTA
    const uint32_t bar_empty = bars + 8 * MAX_STAGES;         // [STAGES]  one set per CTA
    const uint32_t bar_tfull = bars + 16 * MAX_STAGES;        // [2]       one set per CTA
    const uint32_t bar_tempty = bars + 16 * MAX_STAGES + 16;  // [2]       used in the leader CTA
    const uint32_t bar_drain = bars + 16 * MAX_STAGES + 32;   // [1]
    const uint32_t bar_split = bars + 16 * MAX_STAGES + 40;   // [STAGES]  SPLIT only, used in the leader CTA
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + SMEM_RING + SMEM_EPI_OP + SMEM_TABLE + SMEM_BARS);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = (CTAS == 2) ? cluster_ctarank() : 0u;   // 0 = leader
    const uint32_t first_item = (CTAS == 2) ? cluster_id_x() : blockIdx.x;
    const uint32_t item_stride = gridDim.x / CTAS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
            mbar_init(bar_split + 8 * s, 4 * CTAS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, EPI_WARPS * CTAS);
        }
        mbar_init(bar_drain, 1);
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&mapA);
        tma_prefetch_desc(&mapB);
        if (OP != OP_DW) tma_prefetch_desc(&mapC);
    }
    if (warp == 1) {
        if (CTAS == 2) {
            tmem_alloc_pair(smem_u32(tmem_slot), 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    bool ok = true;

    // Work of this CTA (pair).  Two schedules:
    //  * items: work item i = one block with its whole contraction, or one of the nsplit parts of a split block; the
    //    CTA takes items first_item, first_item + item_stride, ...
    //  * units (p.units > 0, small grids whose every block is split): the (block, stage) pairs of the whole launch,
    //    block-major, are dealt out in equal contiguous ranges, one per CTA, so every SM gets the same number of
    //    stages whatever the number of blocks; a range that crosses a block boundary is worked off as two segments.
    // `item` below is the cursor of either schedule; decode() turns it into a block and a stage range and sets the
    // next cursor.  `tile` is the block index in rasterisation order, `partial` says that the segment is only a part
    // of its block's contraction (its result goes to the workspace as fp32 partial sums).
    uint32_t cur_begin = first_item, cur_end = p.total_items;
    if (p.units) {
        cur_begin = (uint32_t)(((uint64_t)first_item * p.units) / item_stride);
        cur_end = (uint32_t)(((uint64_t)(first_item + 1) * p.units) / item_stride);
    }
    uint32_t tile = 0, next_item = 0;
    bool partial = false;
    auto decode = [&](uint32_t item, uint32_t &tr, uint32_t &tc, uint32_t &c_begin, uint32_t &c_end) {
        if (p.units) {
            tile = item / p.nchunks;
            c_begin = item - tile * p.nchunks;
            c_end = min(p.nchunks, c_begin + (cur_end - item));
            partial = true;
            next_item = item + (c_end - c_begin);
        } else {
            uint32_t split = 0;
            if (item < p.n_main) {
                tile = item;
                partial = false;
            } else {
                const uint32_t idx = item - p.n_main, q = idx / p.nsplit;
                tile = p.n_main + q;
                split = idx - q * p.nsplit;
                partial = p.nsplit > 1;
            }
            c_begin = partial ? split * p.chunks_per_split : 0u;
            c_end = partial ? min(p.nchunks, c_begin + p.chunks_per_split) : p.nchunks;
            next_item = item + item_stride;
        }
        uint32_t per_group = p.group_rows * p.tiles_c;
        uint32_t group = tile / per_group, within = tile - group * per_group;
        uint32_t first_r = group * p.group_rows;
        uint32_t gsz = min(p.tiles_r - first_r, p.group_rows);
        tr = first_r + within % gsz;
        tc = within / gsz;
    };

    if (warp == 0) {
        // ===================== producer (both CTAs of a pair) =====================
        uint32_t it = 0;  // stages armed so far
        // transaction bytes of a stage are counted on the leader's barrier
        uint32_t full_base = bar_full;
        if (PAIR_LOADS) full_base = mapa_cluster(bar_full, 0);
        for (uint32_t item = cur_begin; item < cur_end && ok; item = next_item) {
            uint32_t tr, tc, c_begin, c_end;
            decode(item, tr, tc, c_begin, c_end);
            const uint32_t row0 = tr * ITEM_R + rank * TILE_R;     // first output row staged by this CTA (A); row block r adds r * PAIR_R
            const uint32_t col0 = tc * TILE_C + rank * B_COLS;     // first output column staged by this CTA (B)
            for (uint32_t cb = c_begin; cb < c_end && ok; cb += BATCH) {
                const uint32_t nb = min((uint32_t)BATCH, c_end - cb);
                if (OP != OP_DW) {
                    const uint32_t tps = (OP == OP_FWD) ? (uint32_t)B_ATOMS * p.kparts : (uint32_t)B_COLS / p.br;
                    for (uint32_t e = lane; e < nb * tps; e += 32) {
                        const uint32_t ci = e / tps, j = e - ci * tps;
                        uint32_t pk, pn, x_in, y_in;
                        if (OP == OP_FWD) {
                            // box j = (128-byte column block ja, part hh of the stage's contraction rows)
                            const uint32_t ja = j / p.kparts, hh = j - ja * p.kparts;
                            const uint32_t k0 = (cb + ci) * KC + hh * p.br, n = col0 + ja * EPR;
                            pk = k0 / (uint32_t)p.hash.BK;
                            y_in = k0 - pk * (uint32_t)p.hash.BK;
                            pn = n / (uint32_t)p.hash.BN;
                            x_in = n - pn * (uint32_t)p.hash.BN;
                        } else {
                            const uint32_t n0 = (cb + ci) * KC, ko = col0 + j * p.br;
                            pn = n0 / (uint32_t)p.hash.BN;
                            x_in = n0 - pn * (uint32_t)p.hash.BN;
                            pk = ko / (uint32_t)p.hash.BK;
                            y_in = ko - pk * (uint32_t)p.hash.BK;
                        }
                        const uint32_t off = (uint32_t)rz_tile_offset(p.hash, pk, pn);
                        const uint32_t sh = off & (NS - 1);
                        tab_x[ci * MAX_TPS + j] = off - sh + x_in;
                        tab_y[ci * MAX_TPS + j] = y_in;
                        tab_z[ci * MAX_TPS + j] = sh;
                    }
                    __syncwarp();
                }
                if (lane == 0) {
                    for (uint32_t ci = 0; ci < nb; ++ci) {
                        const uint32_t g = it + ci, s = g % STAGES, ph = (g / STAGES) & 1;
                        if (!mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1, RZ_WAIT_SMEM_EMPTY, p.wait, 2000)) {
                            ok = false;
                            it += ci;
                            break;
                        }
                        const uint32_t full = full_base + 8 * s;
                        const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
                        if (PAIR_LOADS) {
                            if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * s, LOAD_BYTES * CTAS);
                        } else {
                            mbar_arrive_expect_tx(bar_full + 8 * s, LOAD_BYTES);
                        }
                        const uint32_t d0 = (cb + ci) * KC;  // contraction start of this stage
                        if (OP == OP_FWD || OP == OP_DX) {
#pragma unroll
                            for (int r = 0; r < RB; ++r) {
                                if (PAIR_LOADS)
                                    tma_load_2d_pair(sa + r * A_BLOCK_BYTES, &mapA, full, (int32_t)d0, (int32_t)(row0 + r * PAIR_R));
                                else
                                    tma_load_2d(sa, &mapA, full, (int32_t)d0, (int32_t)row0);
                            }
                            const uint32_t tps = (OP == OP_FWD) ? (uint32_t)B_ATOMS * p.kparts : (uint32_t)B_COLS / p.br;
                            const uint32_t box_bytes = p.br * 128u;   // (FWD: boxes of one column block are consecutive)
                            for (uint32_t j = 0; j < tps; ++j) {
                                const int32_t x = (int32_t)tab_x[ci * MAX_TPS + j], y = (int32_t)tab_y[ci * MAX_TPS + j],
                                              z = (int32_t)tab_z[ci * MAX_TPS + j];
                                if (PAIR_LOADS) tma_load_3d_pair(sb + j * box_bytes, &mapB, full, x, y, z);
                                else tma_load_3d(sb + j * box_bytes, &mapB, full, x, y, z);
                            }
                        } else {
#pragma unroll
                            for (int r = 0; r < RB; ++r) {
#pragma unroll
                                for (int a = 0; a < A_ATOMS; ++a) {
                                    const uint32_t dst = sa + r * A_BLOCK_BYTES + a * ATOM;
                                    const int32_t x = (int32_t)(row0 + r * PAIR_R + a * EPR);
                                    if (PAIR_LOADS) tma_load_2d_pair(dst, &mapA, full, x, (int32_t)d0);
                                    else tma_load_2d(dst, &mapA, full, x, (int32_t)d0);
                                }
                            }
#pragma unroll
                            for (int j = 0; j < B_ATOMS; ++j) {
                                if (PAIR_LOADS) tma_load_2d_pair(sb + j * ATOM, &mapB, full, (int32_t)(col0 + j * EPR), (int32_t)d0);
                                else tma_load_2d(sb + j * ATOM, &mapB, full, (int32_t)(col0 + j * EPR), (int32_t)d0);
                            }
                        }
                    }
                    if (ok) it += nb;
                }
                __syncwarp();
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                it = __shfl_sync(0xffffffffu, it, 0);
            }
        }
        if (!ok && lane == 0 && (rank == 0 || !PAIR_LOADS)) {
            // give the loads already issued time to land before the CTA retires
            const uint32_t lo = it > STAGES ? it - STAGES : 0;
            for (uint32_t g = lo; g < it; ++g) wait_cycles(bar_full + 8 * (g % STAGES), (g / STAGES) & 1, 4000000);
        }
    } else if (warp == 1) {
        // ===================== MMA issuer (leader CTA only) =====================
        uint32_t it = 0, n_items = 0;
        for (uint32_t item = cur_begin; item < cur_end && ok && rank == 0; item = next_item, ++n_items) {
            uint32_t tr, tc, c_begin, c_end;
            decode(item, tr, tc, c_begin, c_end);
            const uint32_t buf = n_items % NBUF, tph = (n_items / NBUF) & 1;
            if (lane == 0) {
                if (!mbar_wait_bounded(bar_tempty + 8 * buf, tph ^ 1, RZ_WAIT_TMEM_EMPTY, p.wait, 2000)) ok = false;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * RB * TILE_C;
                for (uint32_t c = c_begin; c < c_end && ok; ++c, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded((SPLIT ? bar_split : bar_full) + 8 * s, ph, RZ_WAIT_SMEM_FULL, p.wait)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < MMAS; ++kk) {
                        const uint64_t bd = make_desc_sw128(sb + kk * p.b_kstep, p.b_lbo, p.b_sbo, p.b_layout);
                        const uint32_t acc = (c > c_begin || kk > 0) ? 1u : 0u;
#pragma unroll
                        for (int r = 0; r < RB; ++r) {
                            const uint64_t ad =
                                make_desc_sw128(sa + r * A_BLOCK_BYTES + kk * p.a_kstep, p.a_lbo, p.a_sbo, p.a_layout);
                            if (CTAS == 2) tc_mma_pair<TF32>(d_tmem + r * TILE_C, ad, bd, p.idesc, acc);
                            else tc_mma<TF32>(d_tmem, ad, bd, p.idesc, acc);
                            if (SPLIT) {
                                // + hi(A) * lo(B) + lo(A) * hi(B)
                                const uint64_t ad_lo = make_desc_sw128(sa + LOAD_BYTES + kk * p.a_kstep, p.a_lbo, p.a_sbo, p.a_layout);
                                const uint64_t bd_lo = make_desc_sw128(sb + LOAD_BYTES + kk * p.b_kstep, p.b_lbo, p.b_sbo, p.b_layout);
                                if (CTAS == 2) {
                                    tc_mma_pair<TF32>(d_tmem + CORR_COL, ad, bd_lo, p.idesc, acc);
                                    tc_mma_pair<TF32>(d_tmem + CORR_COL, ad_lo, bd, p.idesc, 1u);
                                } else {
                                    tc_mma<TF32>(d_tmem + CORR_COL, ad, bd_lo, p.idesc, acc);
                                    tc_mma<TF32>(d_tmem + CORR_COL, ad_lo, bd, p.idesc, 1u);
                                }
                            }
                        }
                    }
                    // frees this stage in both CTAs once the MMAs have read it
                    if (CTAS == 2) tc_commit_pair(bar_empty + 8 * s, 3);
                    else tc_commit(bar_empty + 8 * s);
                }
                if (ok) {
                    if (CTAS == 2) tc_commit_pair(bar_tfull + 8 * buf, 3);
                    else tc_commit(bar_tfull + 8 * buf);
                }
            }
            __syncwarp();
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            it = __shfl_sync(0xffffffffu, it, 0);
        }
        if (!ok && lane == 0 && rank == 0) {
            // MMAs may still be running: wait (bounded) until the tensor core has drained
            if (CTAS == 2) tc_commit_pair(bar_drain, 1);
            else tc_commit(bar_drain);
            wait_cycles(bar_drain, 0, 20000000);
        }
    } else if (warp < 2 + EPI_WARPS) {
        // ===================== epilogue (both CTAs; each drains its own 128 rows) =====================
        const uint32_t q = warp & 3;          // TMEM lane quarter this warp may read
        const uint32_t rblk = ((warp - 2) >> 2) % RB;   // which accumulator (row block) of the item this warp drains
        const uint32_t cgrp = ((warp - 2) >> 2) / RB;   // EW > 1: this warp takes the 32-column chunks cgrp, cgrp + EW, ...
        uint32_t own = 0;                                     // mask of those chunks
#pragma unroll
        for (int c2 = 0; c2 < TILE_C / 32; ++c2)
            if (c2 % EW == (int)cgrp) own |= 1u << c2;
        float *scratch = epi_scratch + (warp - 2) * 1024;   // (FWD / DX staging tile; unused by the weight gradient)
        uint32_t tempty_base = bar_tempty;
        if (CTAS == 2) tempty_base = mapa_cluster(bar_tempty, 0);
        uint32_t n_items = 0;
        for (uint32_t item = cur_begin; item < cur_end && ok; item = next_item, ++n_items) {
            uint32_t tr, tc, c_begin, c_end;
            decode(item, tr, tc, c_begin, c_end);
            const uint32_t buf = n_items % NBUF, tph = (n_items / NBUF) & 1;
            const uint32_t rbase = tr * ITEM_R + rblk * PAIR_R + rank * TILE_R + q * 32;   // first row of this warp
            // Weight gradient.  The block is computed TRANSPOSED (A = dY, B = X): an accumulator row (TMEM lane) is an
            // output column n of the virtual weight and an accumulator column is a weight row k.  A thread thus holds,
            // for its n, 32 consecutive k of a chunk, and the 32 lanes of a warp hold 32 consecutive n - which are 32
            // consecutive words of one slice row.  Every reduction instruction is therefore one coalesced 128-byte
            // segment straight out of the registers that tcgen05.ld filled: no transpose through shared memory.
            // A chunk (32 k) lies inside one hash tile (tiles are multiples of 32 both ways).  Chunks of different
            // tiles of one tile column that land on exactly the same addresses (colliding offsets, same rows inside the
            // tile) are summed in registers first, so such a collision costs one set of reductions instead of one
            // per tile.  Lane c (< chunks per block) holds the destination of chunk c.
            uint32_t key_off = 0, key_rel = 0, eqmask = 0, n_rel = 0;
            if (OP == OP_DW) {
                const uint32_t pn = rbase / (uint32_t)p.hash.BN;
                n_rel = rbase - pn * (uint32_t)p.hash.BN;
                if (lane < TILE_C / 32) {
                    const uint32_t kcol = tc * TILE_C + lane * 32, pk = kcol / (uint32_t)p.hash.BK;
                    key_rel = kcol - pk * (uint32_t)p.hash.BK;
                    key_off = (uint32_t)rz_tile_offset(p.hash, pk, pn);
                }
#pragma unroll
                for (int c2 = 0; c2 < TILE_C / 32; ++c2) {
                    const uint32_t o2 = __shfl_sync(0xffffffffu, key_off, c2), r2 = __shfl_sync(0xffffffffu, key_rel, c2);
                    if (o2 == key_off && r2 == key_rel) eqmask |= 1u << c2;
                }
            }
            // (destinations first, then the wait: the hash and the comparisons overlap the block's MMAs)
            // one lane per warp polls (sleeping in the barrier unit between polls); the others wait for it
            bool mine = true;
            if (lane == 0) mine = mbar_wait_bounded(bar_tfull + 8 * buf, tph, RZ_WAIT_TMEM_FULL, p.wait, 20000);
            ok = __shfl_sync(0xffffffffu, (int)mine, 0) != 0;
            if (!ok) break;
            tc_fence_after();
            if (OP == OP_DW && EW > 1 && RB == 1) {
                // Scatter-bound weight gradient.  The warp pulls all its chunks out of TMEM at once and hands the
                // accumulator back before it starts on the reductions, so the next blocks' MMAs never wait for the
                // scatter; loads from TMEM then come in one short burst per block instead of trickling in between
                // the MMAs for the whole epilogue.
                constexpr int NCH = (TILE_C / 32 + EW - 1) / EW;   // chunks per warp
                uint32_t vv[NCH][32];
#pragma unroll
                for (int j = 0; j < NCH; ++j) {
                    const int c = (int)cgrp + j * EW;
                    if (c < TILE_C / 32) tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + buf * TILE_C + c * 32, vv[j]);
                }
#pragma unroll
                for (int j = 0; j < NCH; ++j) tmem_ld_wait_regs(vv[j]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {   // relaxed: a release would wait for the previous block's reductions still in flight
                    if (CTAS == 2) mbar_arrive_cluster_relaxed(tempty_base + 8 * buf);
                    else mbar_arrive_relaxed(bar_tempty + 8 * buf);
                }
                if (rbase >= p.N) continue;
                const bool lane_ok = rbase + lane < p.N;
                const uint32_t bn = (uint32_t)p.hash.BN;
#pragma unroll
                for (int j = 0; j < NCH; ++j) {
                    const int c = (int)cgrp + j * EW;
                    if (c >= TILE_C / 32) break;
                    const uint32_t same = __shfl_sync(0xffffffffu, eqmask, c) & own;
                    if (same & ((1u << c) - 1u)) continue;   // summed into an earlier chunk of this warp
                    const uint32_t kcol = tc * TILE_C + c * 32;
                    uint32_t nk = kcol < p.K ? min(32u, p.K - kcol) : 0u;   // weight rows of this chunk that exist
                    float acc[32];
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[e] = __uint_as_float(vv[j][e]);
#pragma unroll
                    for (int j2 = j + 1; j2 < NCH; ++j2) {
                        const int c2 = (int)cgrp + j2 * EW;
                        if (c2 < TILE_C / 32 && ((same >> c2) & 1u)) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) acc[e] += __uint_as_float(vv[j2][e]);
                            const uint32_t kcol2 = tc * TILE_C + c2 * 32;
                            nk = max(nk, kcol2 < p.K ? min(32u, p.K - kcol2) : 0u);
                        }
                    }
                    const uint32_t off = __shfl_sync(0xffffffffu, key_off, c), rel = __shfl_sync(0xffffffffu, key_rel, c);
                    float *dst = p.dH + off + (uint64_t)rel * bn + n_rel + lane;
                    if (lane_ok) {
                        if (nk == 32) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) atomicAdd(dst + (size_t)e * bn, acc[e] * p.alpha);
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                if ((uint32_t)e < nk) atomicAdd(dst + (size_t)e * bn, acc[e] * p.alpha);
                        }
                    }
                }
                continue;
            }
#pragma nv_diag_suppress 128   // (the one-row-block EW > 1 instantiations never reach the generic chunk loop)
            // FWD / DX: the next chunk streams out of TMEM while this one is converted and stored
            constexpr bool PREFETCH = (OP != OP_DW) && !SPLIT;
            const uint32_t acc_addr = tmem_base + ((q * 32u) << 16) + (buf * RB + rblk) * TILE_C;
            uint32_t vnext[32];
            if (PREFETCH) tmem_ld_32x32(acc_addr + cgrp * 32, vnext);
#pragma unroll 1
            for (int c = (int)cgrp; c < TILE_C / 32; c += EW) {
                uint32_t v[32];
                uint32_t same = 0;
                if (OP == OP_DW) {
                    same = __shfl_sync(0xffffffffu, eqmask, c) & own;   // merge only among this warp's chunks
                    if (same & ((1u << c) - 1u)) continue;   // already merged into an earlier chunk
                }
                if (PREFETCH) {
                    tmem_ld_wait_regs(vnext);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = vnext[j];
                    if (c + EW < TILE_C / 32) tmem_ld_32x32(acc_addr + (c + EW) * 32, vnext);
                } else {
                    tmem_ld_32x32(acc_addr + c * 32, v);
                    tmem_ld_wait();
                }
                if (SPLIT) {   // main + correction accumulators, added with round-to-nearest
                    uint32_t w[32];
                    tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + CORR_COL + c * 32, w);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
                }
                const uint32_t col = tc * TILE_C + c * 32;
                if (OP != OP_DW && p.tma_store && (partial || TF32 || !(c & 1))) {
                    // the staging tile is about to be rewritten: the bulk store issued from it must have read it
                    if (lane == 0) bulk_wait_group_read0();
                    __syncwarp();
                }
                if (OP == OP_DW) {
                    float acc[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(v[j]);
                    uint32_t nk = col < p.K ? min(32u, p.K - col) : 0u;   // weight rows of this chunk that exist
                    uint32_t rest = same & ~((2u << c) - 1u);   // later chunks with the same destination
                    while (rest) {
                        const int c2 = __ffs(rest) - 1;
                        rest &= rest - 1;
                        tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + (buf * RB + rblk) * TILE_C + c2 * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(v[j]);
                        if (SPLIT) {
                            tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + CORR_COL + c2 * 32, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(v[j]);
                        }
                        const uint32_t col2 = tc * TILE_C + c2 * 32;
                        nk = max(nk, col2 < p.K ? min(32u, p.K - col2) : 0u);
                    }
                    const uint32_t off = __shfl_sync(0xffffffffu, key_off, c), rel = __shfl_sync(0xffffffffu, key_rel, c);
                    if (rbase + lane < p.N) {
                        // lane = weight column n, register e = weight row k: one coalesced 128-byte reduction per k
                        float *dst = p.dH + off + (uint64_t)rel * (uint32_t)p.hash.BN + n_rel + lane;
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if ((uint32_t)e < nk) atomicAdd(dst + (size_t)e * (uint32_t)p.hash.BN, acc[e] * p.alpha);
                    }
                } else if (partial) {
                    // split contraction: add the raw fp32 partial sums into this block's ITEM_R x NC workspace tile (a
                    // finalize kernel scales, adds the bias and converts); staged like the store path so every
                    // reduction is a full row segment
                    uint8_t *stage = reinterpret_cast<uint8_t *>(scratch);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        uint4 u;
                        u.x = v[4 * g + 0];
                        u.y = v[4 * g + 1];
                        u.z = v[4 * g + 2];
                        u.w = v[4 * g + 3];
                        *reinterpret_cast<uint4 *>(stage + lane * 128 + ((g ^ (lane & 7)) * 16)) = u;
                    }
                    __syncwarp();
                    const uint32_t cc = lane & 7, ccol = col + cc * 4;
                    float *wtile = p.ws + (size_t)(tile - p.n_main) * (ITEM_R * NC) +
                                   (size_t)(rbase - tr * ITEM_R) * NC + (c * 32 + cc * 4);
#pragma unroll
                    for (int it4 = 0; it4 < 8; ++it4) {
                        const uint32_t rr = it4 * 4 + (lane >> 3);
                        const uint4 u = *reinterpret_cast<const uint4 *>(stage + rr * 128 + ((cc ^ (rr & 7)) * 16));
                        const uint32_t grow = rbase + rr;
                        if (grow < p.rows && ccol < p.cols)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(wtile + (size_t)rr * NC),
                                         "f"(__uint_as_float(u.x)), "f"(__uint_as_float(u.y)), "f"(__uint_as_float(u.z)),
                                         "f"(__uint_as_float(u.w))
                                         : "memory");
                    }
                    __syncwarp();
                } else {
                    // scale (+ bias, ReLU), convert, and stage this lane's row segment in shared memory in
                    // 16-byte chunks (chunk index XOR row keeps both phases bank-conflict free); once a
                    // 128-byte row segment is complete the warp writes it out 4 full rows per instruction.
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
                    if (OP == OP_FWD) {
                        if (p.bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < p.cols) f[j] += __ldg(p.bias + col + j);
                        }
                        if (p.relu) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = fmaxf(f[j], 0.f);
                        }
                    }
                    uint8_t *stage = reinterpret_cast<uint8_t *>(scratch);
                    constexpr int CHUNKS_PER_LD = TF32 ? 8 : 4;          // 16-byte chunks produced per 32 columns
                    const int cbase = TF32 ? 0 : (c & 1) * 4;             // bf16: two loads fill one 128-byte row
#pragma unroll
                    for (int g = 0; g < CHUNKS_PER_LD; ++g) {
                        uint4 u;
                        if (TF32) {
                            u.x = __float_as_uint(f[4 * g + 0]);
                            u.y = __float_as_uint(f[4 * g + 1]);
                            u.z = __float_as_uint(f[4 * g + 2]);
                            u.w = __float_as_uint(f[4 * g + 3]);
                        } else {
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(f[8 * g + 0], f[8 * g + 1]);
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(f[8 * g + 2], f[8 * g + 3]);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(f[8 * g + 4], f[8 * g + 5]);
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(f[8 * g + 6], f[8 * g + 7]);
                            u.x = *reinterpret_cast<uint32_t *>(&h0);
                            u.y = *reinterpret_cast<uint32_t *>(&h1);
                            u.z = *reinterpret_cast<uint32_t *>(&h2);
                            u.w = *reinterpret_cast<uint32_t *>(&h3);
                        }
                        *reinterpret_cast<uint4 *>(stage + lane * 128 + (((cbase + g) ^ (lane & 7)) * 16)) = u;
                    }
                    if ((TF32 || (c & 1)) && p.tma_store) {
                        // one bulk tensor store per staged 32-row x 128-byte tile (the tile is in the 128-byte-swizzle
                        // layout the store expects; rows and columns past the matrix edge are clipped by the unit)
                        const uint32_t col_seg = TF32 ? col : col - 32;
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0 && rbase < p.rows && col_seg < p.cols) {
                            tma_store_2d(&mapC, smem_u32(stage), (int32_t)col_seg, (int32_t)rbase);
                            bulk_commit_group();
                        }
                    } else if (TF32 || (c & 1)) {
                        __syncwarp();
                        constexpr int EPC = TF32 ? 4 : 8;                 // elements per 16-byte chunk
                        const uint32_t col_seg = TF32 ? col : col - 32;   // first column of the staged 128-byte segment
                        const uint32_t cc = lane & 7, ccol = col_seg + cc * EPC;
#pragma unroll
                        for (int it4 = 0; it4 < 8; ++it4) {
                            const uint32_t rr = it4 * 4 + (lane >> 3);
                            const uint4 u = *reinterpret_cast<const uint4 *>(stage + rr * 128 + ((cc ^ (rr & 7)) * 16));
                            const uint32_t grow = rbase + rr;
                            if (grow < p.rows && ccol < p.cols)
                                *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) +
                                                           ((size_t)grow * p.cols + ccol) * (TF32 ? 4 : 2)) = u;
                        }
                        __syncwarp();
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2) mbar_arrive_cluster(tempty_base + 8 * buf);
                else mbar_arrive(bar_tempty + 8 * buf);
            }
        }
        if (OP != OP_DW && lane == 0) bulk_wait_group0();   // bulk stores still in flight read this CTA's shared memory
    }

    else if (SPLIT) {
        // ===================== splitter (SPLIT only): hi/lo parts of every staged tile =====================
        const uint32_t tid = threadIdx.x - (2 + EPI_WARPS) * 32;   // 0..127
        uint32_t split_base = bar_split;
        if (CTAS == 2) split_base = mapa_cluster(bar_split, 0);
        uint32_t it = 0;
        for (uint32_t item = cur_begin; item < cur_end && ok; item = next_item) {
            uint32_t tr, tc, c_begin, c_end;
            decode(item, tr, tc, c_begin, c_end);
            for (uint32_t c = c_begin; c < c_end && ok; ++c, ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                bool mine = mbar_wait_bounded(bar_full + 8 * s, ph, RZ_WAIT_SMEM_FULL, p.wait, 1000);
                ok = __all_sync(0xffffffffu, mine);
                if (!ok) break;
                uint4 *hi = reinterpret_cast<uint4 *>(smem_gen + s * STAGE_BYTES);
                uint4 *lo = reinterpret_cast<uint4 *>(smem_gen + s * STAGE_BYTES + LOAD_BYTES);
#pragma unroll 4
                for (uint32_t v = tid; v < LOAD_BYTES / 16; v += 128) {
                    uint4 x = hi[v], h, l;
                    h.x = x.x & 0xFFFFE000u;
                    h.y = x.y & 0xFFFFE000u;
                    h.z = x.z & 0xFFFFE000u;
                    h.w = x.w & 0xFFFFE000u;
                    l.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(h.x));
                    l.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(h.y));
                    l.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(h.z));
                    l.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(h.w));
                    hi[v] = h;
                    lo[v] = l;
                }
                fence_proxy_async();   // the tensor core reads these tiles through the async proxy
                __syncwarp();
                if (lane == 0) {
                    if (CTAS == 2) mbar_arrive_cluster(split_base + 8 * s);
                    else mbar_arrive(bar_split + 8 * s);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();   // neither CTA retires while the peer may still signal or read it
    if (warp == 1) {
        tc_fence_after();
        __syncwarp();
        if (CTAS == 2) tmem_dealloc_pair(tmem_base, 512);
        else tmem_dealloc(tmem_base, 512);
    }
}

// ---- self-test of the bounded-wait machinery ---------------------------------------------------
// One thread waits on an mbarrier that nothing will ever complete.  The wait must give up after
// `limit` cycles, leave its code in the status word and let the kernel return normally.
__global__ void rz_wait_selftest_kernel(WaitCtx w)
{
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
        (void)mbar_wait_bounded(smem_u32(&bar), 0, RZ_WAIT_SELFTEST, w);
    }
}

// ---- shadow copies and SGD -----------------------------------------------------------------

__device__ __forceinline__ uint32_t to_tf32(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

// copy s, element j  =  convert(hashed[j + s])   (0 past the end); one thread writes NS elements of every copy
// `raw` (fp32 elements only): keep every mantissa bit, for the split-precision kernels that form hi/lo themselves
template <bool TF32>
__global__ void rz_shadow_kernel(const float *__restrict__ hashed, uint8_t *__restrict__ shadow, uint32_t H, uint32_t Hc,
                                 size_t copy_stride, int raw)
{
    constexpr int NS = TF32 ? 4 : 8;
    const uint32_t groups = Hc / NS;
    for (uint32_t g = blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += gridDim.x * blockDim.x) {
        const uint32_t j0 = g * NS;
        float v[2 * NS];
#pragma unroll
        for (int i = 0; i < 2 * NS; ++i) v[i] = (j0 + i < H) ? hashed[j0 + i] : 0.f;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            uint4 u;
            if (TF32) {
                u.x = raw ? __float_as_uint(v[s + 0]) : to_tf32(v[s + 0]);
                u.y = raw ? __float_as_uint(v[s + 1]) : to_tf32(v[s + 1]);
                u.z = raw ? __float_as_uint(v[s + 2]) : to_tf32(v[s + 2]);
                u.w = raw ? __float_as_uint(v[s + 3]) : to_tf32(v[s + 3]);
            } else {
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[s + 0], v[s + 1]);
                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[s + 2], v[s + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[s + 4], v[s + 5]);
                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[s + 6], v[s + 7]);
                u.x = *reinterpret_cast<uint32_t *>(&h0);
                u.y = *reinterpret_cast<uint32_t *>(&h1);
                u.z = *reinterpret_cast<uint32_t *>(&h2);
                u.w = *reinterpret_cast<uint32_t *>(&h3);
            }
            *reinterpret_cast<uint4 *>(shadow + s * copy_stride + (size_t)g * 16) = u;
        }
    }
}

__global__ void rz_sgd_kernel(float *__restrict__ hashed, const float *__restrict__ dH, float lr, uint32_t H)
{
    const uint32_t n4 = H / 4;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
        float4 h = reinterpret_cast<float4 *>(hashed)[i];
        const float4 g = reinterpret_cast<const float4 *>(dH)[i];
        h.x -= lr * g.x;
        h.y -= lr * g.y;
        h.z -= lr * g.z;
        h.w -= lr * g.w;
        reinterpret_cast<float4 *>(hashed)[i] = h;
    }
    if (blockIdx.x == 0 && threadIdx.x < (H & 3u)) {
        const uint32_t i = n4 * 4 + threadIdx.x;
        hashed[i] -= lr * dH[i];
    }
}

// v = momentum * v + dH;  hashed -= lr * v   (heavy-ball SGD on the hashed array)
__global__ void rz_sgd_momentum_kernel(float *__restrict__ hashed, const float *__restrict__ dH, float *__restrict__ vel,
                                       float lr, float momentum, uint32_t H)
{
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) {
        const float v = momentum * vel[i] + dH[i];
        vel[i] = v;
        hashed[i] -= lr * v;
    }
}

// The optimiser step and the shadow refresh in ONE pass over the hashed array:
//   (velocity = momentum * velocity + dH;)   hashed -= lr * (velocity | dH);   copy s, element j = convert(hashed[j + s]).
// A thread owns one aligned group of NS elements: it updates them in place and writes the NS 16-byte pieces of the
// shifted copies that start in its group.  Those pieces reach NS - 1 elements into the NEXT group, whose new values
// come from the neighbouring lane (shuffle) or warp (shared memory) of the same chunk of SGD_CHUNK groups.  The last group of
// a chunk has its neighbour in another block, which may or may not have updated it yet: its pieces for copies
// 1 .. NS-1 are left to the block that finishes last (a ticket counter tells which), which by then reads final values.
constexpr int SGD_CHUNK = 1024;    // groups per block iteration (= threads per block): few chunk boundaries for the last block
constexpr int SGD_TICKETS = 64;    // launches that may be in flight at once, one ticket word each
__device__ unsigned g_sgd_ticket[SGD_TICKETS];

template <bool TF32>
__device__ __forceinline__ uint4 shadow_piece(const float *v, int raw)
{
    uint4 u;
    if (TF32) {
        u.x = raw ? __float_as_uint(v[0]) : to_tf32(v[0]);
        u.y = raw ? __float_as_uint(v[1]) : to_tf32(v[1]);
        u.z = raw ? __float_as_uint(v[2]) : to_tf32(v[2]);
        u.w = raw ? __float_as_uint(v[3]) : to_tf32(v[3]);
    } else {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
        u.x = *reinterpret_cast<uint32_t *>(&h0);
        u.y = *reinterpret_cast<uint32_t *>(&h1);
        u.z = *reinterpret_cast<uint32_t *>(&h2);
        u.w = *reinterpret_cast<uint32_t *>(&h3);
    }
    return u;
}

template <bool TF32, bool MOMENTUM>
__global__ void __launch_bounds__(SGD_CHUNK)
rz_sgd_shadow_kernel(float *__restrict__ hashed, const float *__restrict__ dH, float *__restrict__ vel, float lr, float momentum,
                     uint8_t *__restrict__ shadow, uint32_t H, uint32_t Hc, size_t copy_stride, int raw, unsigned *ticket)
{
    constexpr int NS = TF32 ? 4 : 8;
    __shared__ float first_of_warp[SGD_CHUNK / 32][NS];
    __shared__ bool is_last;
    const uint32_t groups = Hc / NS, nchunks = (groups + SGD_CHUNK - 1) / SGD_CHUNK;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t chunk = blockIdx.x; chunk < nchunks; chunk += gridDim.x) {
        const uint32_t g = chunk * SGD_CHUNK + threadIdx.x, j0 = g * NS;
        float nv[2 * NS];   // new values of this group, then of the next one
#pragma unroll
        for (int i = 0; i < NS; ++i) nv[i] = 0.f;
        if (g < groups && j0 < H) {
            if (j0 + NS <= H) {
#pragma unroll
                for (int q = 0; q < NS / 4; ++q) {
                    float4 h = reinterpret_cast<float4 *>(hashed + j0)[q];
                    float4 d = reinterpret_cast<const float4 *>(dH + j0)[q];
                    if (MOMENTUM) {
                        const float4 v = reinterpret_cast<float4 *>(vel + j0)[q];
                        d.x = momentum * v.x + d.x, d.y = momentum * v.y + d.y, d.z = momentum * v.z + d.z, d.w = momentum * v.w + d.w;
                        reinterpret_cast<float4 *>(vel + j0)[q] = d;
                    }
                    h.x -= lr * d.x, h.y -= lr * d.y, h.z -= lr * d.z, h.w -= lr * d.w;
                    reinterpret_cast<float4 *>(hashed + j0)[q] = h;
                    nv[4 * q + 0] = h.x, nv[4 * q + 1] = h.y, nv[4 * q + 2] = h.z, nv[4 * q + 3] = h.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    if (j0 + i < H) {
                        float d = dH[j0 + i];
                        if (MOMENTUM) {
                            d = momentum * vel[j0 + i] + d;
                            vel[j0 + i] = d;
                        }
                        nv[i] = hashed[j0 + i] - lr * d;
                        hashed[j0 + i] = nv[i];
                    }
                }
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < NS; ++i) first_of_warp[warp][i] = nv[i];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NS; ++i) nv[NS + i] = __shfl_down_sync(0xffffffffu, nv[i], 1);
        const bool chunk_end = threadIdx.x == SGD_CHUNK - 1;
        if (lane == 31 && !chunk_end) {
#pragma unroll
            for (int i = 0; i < NS; ++i) nv[NS + i] = first_of_warp[warp + 1][i];
        }
        const bool deferred = chunk_end && g + 1 < groups;   // the neighbour group belongs to another block
        if (chunk_end) {
#pragma unroll
            for (int i = 0; i < NS; ++i) nv[NS + i] = 0.f;   // (past the end of the array when not deferred)
        }
        if (g < groups) {
#pragma unroll
            for (int s2 = 0; s2 < NS; ++s2)
                if (s2 == 0 || !deferred)
                    *reinterpret_cast<uint4 *>(shadow + s2 * copy_stride + (size_t)g * 16) = shadow_piece<TF32>(nv + s2, raw);
        }
        __syncthreads();   // first_of_warp is rewritten by the next chunk
    }
    // the block that finishes last fills in the pieces that straddle chunk boundaries
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (uint32_t b = threadIdx.x; b + 1 < nchunks; b += SGD_CHUNK) {
        const uint32_t g = b * SGD_CHUNK + SGD_CHUNK - 1, j0 = g * NS;
        float nv[2 * NS];
#pragma unroll
        for (int i = 0; i < 2 * NS; ++i) nv[i] = (j0 + i < H) ? __ldcg(hashed + j0 + i) : 0.f;
#pragma unroll
        for (int s2 = 1; s2 < NS; ++s2)
            *reinterpret_cast<uint4 *>(shadow + s2 * copy_stride + (size_t)g * 16) = shadow_piece<TF32>(nv + s2, raw);
    }
    if (threadIdx.x == 0) *ticket = 0;   // ready for the next launch that draws this ticket word
}

// out = convert(alpha * partial_sums (+ bias) (ReLU)) for the blocks of a FWD / DX launch whose contraction was
// split: block n_main + i owns workspace tile i (item_r x nc floats, row-major); gridDim.y CTAs share a block.
struct FinalizeGeom {
    uint32_t rows, cols, item_r, nc, tiles_r, tiles_c, group_rows, n_main, n_tiles;
};

template <typename T>
__global__ void rz_finalize_kernel(const float *__restrict__ ws, T *__restrict__ out, const float *__restrict__ bias,
                                   FinalizeGeom g, float alpha, int relu)
{
    const uint32_t quads_per_row = g.nc / 4;
    for (uint32_t i = blockIdx.x; i + g.n_main < g.n_tiles; i += gridDim.x) {
        const uint32_t tile = g.n_main + i;
        const uint32_t per_group = g.group_rows * g.tiles_c;
        const uint32_t group = tile / per_group, within = tile - group * per_group;
        const uint32_t first_r = group * g.group_rows;
        const uint32_t gsz = min(g.tiles_r - first_r, g.group_rows);
        const uint32_t tr = first_r + within % gsz, tc = within / gsz;
        const float *wt = ws + (size_t)i * g.item_r * g.nc;
        const uint32_t valid_rows = min(g.item_r, g.rows - tr * g.item_r);   // rows of the block that exist
        const uint32_t nq = valid_rows * quads_per_row;
        for (uint32_t e = blockIdx.y * blockDim.x + threadIdx.x; e < nq; e += blockDim.x * gridDim.y) {
            const uint32_t lr = e / quads_per_row, lc = (e - lr * quads_per_row) * 4;
            const uint32_t row = tr * g.item_r + lr, col = tc * g.nc + lc;
            if (row >= g.rows || col >= g.cols) continue;   // cols is a multiple of 4
            float4 v = *reinterpret_cast<const float4 *>(wt + (size_t)lr * g.nc + lc);
            v.x *= alpha, v.y *= alpha, v.z *= alpha, v.w *= alpha;
            if (bias) v.x += bias[col], v.y += bias[col + 1], v.z += bias[col + 2], v.w += bias[col + 3];
            if (relu) v.x = fmaxf(v.x, 0.f), v.y = fmaxf(v.y, 0.f), v.z = fmaxf(v.z, 0.f), v.w = fmaxf(v.w, 0.f);
            const size_t o = (size_t)row * g.cols + col;
            if (sizeof(T) == 4) {
                *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + o) = v;
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                uint2 u;
                u.x = *reinterpret_cast<uint32_t *>(&lo);
                u.y = *reinterpret_cast<uint32_t *>(&hi);
                *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(out) + o) = u;
            }
        }
    }
}

// ---- host side -----------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

struct Geometry {
    int es, epr, ns;
    uint32_t Hc;
    size_t copy_stride;
};

Geometry geometry(const rz_problem *pb)
{
    Geometry g;
    const bool tf32 = pb->precision != RZ_PREC_BF16;   // fp32 elements (tf32 and split-precision fp32)
    g.es = tf32 ? 4 : 2;
    g.epr = 128 / g.es;
    g.ns = 16 / g.es;
    g.Hc = (uint32_t)((pb->H + 63) / 64 * 64);
    g.copy_stride = ((size_t)g.Hc * g.es + 255) / 256 * 256;
    return g;
}

// `mn_major`: the tile feeds an M/N-major operand; for 32-bit elements that needs the 32-byte-chunk flavour
// of the 128-byte swizzle, every other case uses the 16-byte-chunk one.
// Encoded maps are pure functions of (base, type, swizzle flavour, extents, strides, box): each host thread keeps
// the last few it made, so steady-state launches (the same tensors step after step) encode nothing.
struct MapKey {
    const void *base;
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    int rank, tf32, mn_major;
    bool operator==(const MapKey &o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapCache {
    static constexpr int N = 16;
    MapKey key[N];
    alignas(64) CUtensorMap map[N];
    int used = 0, next = 0;
};

int encode(CUtensorMap *map, bool tf32, bool mn_major, void *base, int rank, const uint64_t *dims,
           const uint64_t *strides_bytes, const uint32_t *box)
{
    static thread_local MapCache cache;
    MapKey k;
    memset(&k, 0, sizeof(k));   // (padding too: keys are compared bytewise)
    k.base = base, k.rank = rank, k.tf32 = tf32, k.mn_major = mn_major;
    for (int i = 0; i < rank; ++i) k.dims[i] = dims[i], k.box[i] = box[i];
    for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides_bytes[i];
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == k) {
            *map = cache.map[i];
            return RZ_OK;
        }
    EncodeTiledFn fn = get_encode();
    if (!fn) return rz_record_cuda(cudaErrorUnknown, "cuTensorMapEncodeTiled not available");
    // The encoder is a driver call and wants a context current on this thread.  A thread that has made no
    // runtime call yet (an autograd worker, say) has none: a null free binds the device's primary context.
    static thread_local bool bound = false;
    if (!bound) {
        int st = rz_record_cuda(cudaFree(nullptr), "bind the primary context");
        if (st) return st;
        bound = true;
    }
    cuuint64_t gdim[3];
    cuuint64_t gstr[2];
    cuuint32_t bx[3], estr[3];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        estr[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    CUresult r = fn(map, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, base,
                    gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    (tf32 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[96];
        snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed (CUresult %d, rank %d)", (int)r, rank);
        return rz_record_cuda(cudaErrorInvalidValue, msg);
    }
    const int slot = cache.used < MapCache::N ? cache.used++ : (cache.next = (cache.next + 1) % MapCache::N);
    cache.key[slot] = k;
    cache.map[slot] = *map;
    return RZ_OK;
}

int num_sms()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// SMs a launch may occupy: all of them, less the ones the problem asks to leave idle (a collective that should
// run beside a persistent kernel needs SMs of its own); never fewer than two.
int usable_sms(const rz_problem *pb)
{
    int n = num_sms() - (pb->sm_reserve > 0 ? pb->sm_reserve : 0);
    return n < 2 ? 2 : n;
}

uint32_t env_u32(const char *name, uint32_t dflt)
{
    const char *s = getenv(name);
    return s ? (uint32_t)strtoul(s, nullptr, 0) : dflt;
}

// Bring-up / A-B knobs, read from the environment once (rz_reload_env() reads them again):
//   RZ_TC_CONFIG 1..5 forces a block shape, RZ_TC_NOSPLIT=1 turns contraction splitting off, RZ_TC_EW_STAGES is the
//   longest contraction (stages) that gets the sixteen-warp weight-gradient epilogue, RZ_TC_GROUP the rasterisation
//   group (row tiles), RZ_TC_TMA_STORE=0 plain stores instead of bulk tensor stores, RZ_TC_VERBOSE=1 one line per launch,
//   RZ_TC_UNIT_RANGES=0 keeps fully split launches on nsplit equal parts per block instead of equal stage ranges,
//   RZ_TC_DW_EW2=0 gives the two-row-block weight gradient eight epilogue warps instead of sixteen.
struct Knobs {
    std::atomic<uint32_t> config{0}, no_split{0}, ew_stages{64}, group{0}, tma_store{1}, verbose{0}, unit_ranges{1}, dw_ew2{1};
    std::atomic<bool> ready{false};
};
Knobs g_knobs;

void load_knobs()
{
    g_knobs.config.store(env_u32("RZ_TC_CONFIG", 0));
    g_knobs.no_split.store(env_u32("RZ_TC_NOSPLIT", 0));
    g_knobs.ew_stages.store(env_u32("RZ_TC_EW_STAGES", 64));
    g_knobs.group.store(env_u32("RZ_TC_GROUP", 0));
    g_knobs.tma_store.store(env_u32("RZ_TC_TMA_STORE", 1));
    g_knobs.verbose.store(env_u32("RZ_TC_VERBOSE", 0));
    g_knobs.unit_ranges.store(env_u32("RZ_TC_UNIT_RANGES", 1));
    g_knobs.dw_ew2.store(env_u32("RZ_TC_DW_EW2", 1));
    g_knobs.ready.store(true, std::memory_order_release);
}

const Knobs &knobs()
{
    if (!g_knobs.ready.load(std::memory_order_acquire)) load_knobs();
    return g_knobs;
}

// Block shape of a launch.  (ctas, rb, nc): CTAs per block (2 = cluster pair driving cta_group::2 MMAs), row
// blocks per pair, block columns.  Blocks are rows = 128*ctas*rb by nc.
struct TcConfig {
    int ctas, rb, nc;
    int nsplit;   // parts the contraction of the blocks from n_main on is split into (1 = no block is split)
    int n_main;   // blocks [0, n_main) keep their whole contraction; 0 with nsplit > 1 = every block is split
    int ew;       // epilogue warps per TMEM lane quarter (0 or 1 = one; 4 = weight gradient of a short contraction)
};

// Candidates from the largest block down, with the relative tensor throughput each sustains when the grid
// fills the machine (the wide pair blocks move the fewest L2 bytes per flop; narrow single-CTA blocks are
// L2-bound but keep every SM busy on small grids).
const struct {
    TcConfig cfg;
    double speed;
} kCandidates[] = {
    {{2, 2, 256, 1, 0}, 1.00}, {{2, 1, 256, 1, 0}, 0.80}, {{1, 1, 256, 1, 0}, 0.58}, {{1, 1, 128, 1, 0}, 0.40}, {{1, 1, 64, 1, 0}, 0.25},
};

// Pick the block shape with the best (occupancy of the last wave) x (shape throughput), among the shapes the
// problem allows.  RZ_TC_CONFIG = 1..5 forces one shape (1 = 128x256 single CTA,
// 2 = pair 256x256, 3 = pair 512x256, 4 = single 128x128, 5 = single 128x64).
TcConfig choose_config(const rz_problem *pb, int op)
{
    const bool bf16 = pb->precision == RZ_PREC_BF16;
    const bool split = pb->precision == RZ_PREC_FP32;
    const int64_t rows = (op == RZ_OP_BACKWARD_WEIGHT) ? pb->N : pb->M;   // (weight gradient: transposed block, N x K)
    const int64_t cols = (op == RZ_OP_FORWARD) ? pb->N : pb->K;
    const int64_t depth = (op == RZ_OP_FORWARD) ? pb->K : (op == RZ_OP_BACKWARD_INPUT ? pb->N : pb->M);
    const int64_t stages = (depth + (bf16 ? 63 : 31)) / (bf16 ? 64 : 32);
    const int sms = usable_sms(pb);
    auto allowed = [&](const TcConfig &c) {
        if (split && c.rb == 2) return false;                       // split precision has no two-row-block variant
        // with two row blocks the epilogue cannot overlap the next main loop: the contraction must amortise it
        // (the weight gradient's scatter epilogue is several times as long as a store epilogue; measured: at 32 stages
        // the one-row-block pair with sixteen epilogue warps is 4 % ahead, at 64 stages two row blocks are 6 % ahead)
        if (c.rb == 2 && stages < (op == RZ_OP_BACKWARD_WEIGHT ? 48 : 12)) return false;
        const int64_t bcols = c.nc / c.ctas;                        // whole B boxes per hash tile (input gradient)
        if (op == RZ_OP_BACKWARD_INPUT && (pb->BK <= bcols ? bcols % pb->BK != 0 : pb->BK % bcols != 0)) return false;
        return true;
    };
    // Small grids: split the contraction over several blocks so that every SM has work.  The weight gradient adds
    // its partial blocks straight into the hashed gradient; FWD / DX add fp32 partials into a workspace that a
    // finalize kernel scales and converts (two more small launches, so only contractions of 64 stages or more are
    // split).  At least 16 pipeline stages per part.
    auto split_for = [&](int64_t items, int64_t slots) {
        if (items * 2 > slots) return (int64_t)1;
        if (op != RZ_OP_BACKWARD_WEIGHT && stages < 64) return (int64_t)1;
        int64_t want = slots / items, most = stages / (op == RZ_OP_BACKWARD_WEIGHT ? 8 : 16);
        if (most < 1) most = 1;
        return want < most ? want : most;
    };
    const uint32_t forced = knobs().config.load(std::memory_order_relaxed);
    const bool no_split = knobs().no_split.load(std::memory_order_relaxed) != 0;
    TcConfig best = kCandidates[4].cfg;
    double best_score = -1.0;
    for (int i = 0; i < 5; ++i) {
        const auto &cand = kCandidates[i];
        TcConfig c = cand.cfg;
        if (!allowed(c)) continue;
        const int64_t block_rows = (int64_t)TILE_R * c.ctas * c.rb;
        const int64_t items = ((rows + block_rows - 1) / block_rows) * ((cols + c.nc - 1) / c.nc);
        const int64_t slots = sms / c.ctas;
        if (!no_split) c.nsplit = (int)split_for(items, slots);
        if (split) {   // bound the accumulation chains of split precision: at most 2048 contraction elements per part
            const int64_t need = (depth + 2047) / 2048;
            if (c.nsplit < need) c.nsplit = (int)need;
        }
        // Ragged last wave: the blocks left over after the full waves are split along the contraction, so the tail costs
        // ceil(tail * parts / slots) / parts of a wave instead of a whole one.  Every part pays the block's epilogue
        // again (FWD / DX: fp32 reductions into the workspace, which only those blocks go through, plus the finalize
        // launch; DW: its scatter, which it pays anyway), counted here in pipeline stages.
        const int64_t tail = items % slots;
        double tail_waves = 1.0;   // time of the last wave, in whole-contraction blocks
        if (!no_split && c.nsplit == 1 && items > slots && tail > 0 && stages >= 32) {
            const bool dw = op == RZ_OP_BACKWARD_WEIGHT;
            const double per_part = dw ? (c.rb == 2 ? 19.0 : 4.0) : (c.rb == 2 ? 10.0 : 5.0);
            const double whole = (double)stages + (dw ? per_part : 0.0);
            int64_t best_parts = 1;
            const int64_t most = stages / 8 < 16 ? stages / 8 : 16;
            for (int64_t parts = 2; parts <= most; ++parts) {
                const double t = (double)((tail * parts + slots - 1) / slots) * ((double)stages / (double)parts + per_part) / whole +
                                 (dw ? 0.0 : 0.05);
                if (t < tail_waves - 0.04) {
                    tail_waves = t;
                    best_parts = parts;
                }
            }
            if (best_parts > 1) {
                c.nsplit = (int)best_parts;
                c.n_main = (int)(items - tail);
            }
        }
        // Weight gradient of a short contraction: the scatter epilogue (one reduction per 32 elements, issued by
        // one warp per scheduler) outlasts the main loop; sixteen epilogue warps hide its instruction latency.
        if (op == RZ_OP_BACKWARD_WEIGHT && !split && c.rb == 1 && stages / c.nsplit <= (int64_t)knobs().ew_stages.load(std::memory_order_relaxed))
            c.ew = 4;
        // Two row blocks: the scatter cannot overlap the next block's MMAs, so it should at least be short - sixteen
        // epilogue warps (two per TMEM lane quarter and row block) keep twice as many reductions in flight as eight.
        if (op == RZ_OP_BACKWARD_WEIGHT && !split && c.rb == 2 && knobs().dw_ew2.load(std::memory_order_relaxed)) c.ew = 2;
        if (forced >= 1 && forced <= 5) {
            static const int order[5] = {2, 1, 0, 3, 4};
            if (order[forced - 1] == i) return c;
            continue;
        }
        if (rows < block_rows / 2 && c.ctas * c.rb > 1) continue;   // do not pair CTAs over rows that do not exist
        // time in waves of whole-contraction blocks, against the ideal items / slots
        double waves;
        if (c.nsplit == 1) {
            waves = (double)((items + slots - 1) / slots);
        } else if (c.n_main == 0) {
            waves = (double)((items * c.nsplit + slots - 1) / slots) / c.nsplit + 0.1;
        } else {
            waves = (double)(c.n_main / slots) + tail_waves;
        }
        const double occupancy = ((double)items / (double)slots) / waves;
        // useful fraction of the block (ragged last row block)
        const double fill = (double)rows / (double)(((rows + block_rows - 1) / block_rows) * block_rows);
        const double score = (occupancy > 1.0 ? 1.0 : occupancy) * fill * cand.speed;
        if (score > best_score * 1.02) {   // prefer the larger block on near ties
            best_score = score;
            best = c;
        }
    }
    return best;
}

// fp32 partial-sum workspace a FWD / DX launch with split blocks needs: one block-sized tile per split block
// (0 for whole-contraction launches and for DW, which adds its parts straight into the hashed gradient)
size_t workspace_bytes(const rz_problem *pb, int op)
{
    if (op == RZ_OP_BACKWARD_WEIGHT) return 0;
    const TcConfig c = choose_config(pb, op);
    if (c.nsplit <= 1) return 0;
    const int64_t cols = (op == RZ_OP_BACKWARD_INPUT) ? pb->K : pb->N;
    const int64_t block_rows = (int64_t)TILE_R * c.ctas * c.rb;
    const int64_t items = ((pb->M + block_rows - 1) / block_rows) * ((cols + c.nc - 1) / c.nc);
    return (size_t)(items - c.n_main) * (size_t)block_rows * (size_t)c.nc * sizeof(float);
}

uint32_t dx_box_rows(const rz_problem *pb, const TcConfig &c)
{
    const uint32_t bcols = (uint32_t)(c.nc / c.ctas);
    return (uint32_t)pb->BK < bcols ? (uint32_t)pb->BK : bcols;
}

// FWD: slice rows per B box - a stage's contraction rows, or one hash tile of them when tiles are shorter
uint32_t fwd_box_rows(const rz_problem *pb)
{
    const uint32_t kc = pb->precision == RZ_PREC_BF16 ? 64u : 32u;
    return (uint32_t)pb->BK < kc ? (uint32_t)pb->BK : kc;
}

template <int OP, bool TF32, int CTAS, int RB, int SPLIT, int NC, int EW = 1>
int launch_tc(const RzLaunchCtx &c, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC, TcParams &p,
              const TcConfig &plan)
{
    const rz_problem *pb = c.pb;
    constexpr int ES = TF32 ? 4 : 2;
    constexpr int EPR = 128 / ES;
    constexpr int KC = EPR;
    constexpr int PAIR_R = TILE_R * CTAS;
    constexpr int ITEM_R = PAIR_R * RB;
    constexpr int NTHREADS = num_threads(RB, SPLIT, EW);
    constexpr int STAGES_HOST = num_stages(OP, CTAS, RB, SPLIT, NC, EW);
    p.hash = c.hash;
    p.M = (uint32_t)pb->M;
    p.K = (uint32_t)pb->K;
    p.N = (uint32_t)pb->N;
    p.rows = (OP == OP_DW) ? p.N : p.M;                  // (the weight gradient is computed transposed: N x K)
    p.cols = (OP == OP_FWD) ? p.N : p.K;
    const uint32_t depth = (OP == OP_FWD) ? p.K : (OP == OP_DX ? p.N : p.M);
    p.tiles_r = (p.rows + ITEM_R - 1) / ITEM_R;
    p.tiles_c = (p.cols + NC - 1) / NC;
    p.nchunks = (depth + KC - 1) / KC;
    p.br = OP == OP_FWD ? fwd_box_rows(pb) : dx_box_rows(pb, TcConfig{CTAS, RB, NC});
    p.kparts = KC / fwd_box_rows(pb);
    p.group_rows = knobs().group.load(std::memory_order_relaxed);
    if (p.group_rows < 1) p.group_rows = GROUP_ROWS / RB;

    auto kern = rz_tc_kernel<OP, TF32, CTAS, RB, SPLIT, NC, EW>;
    constexpr int SMEM_TOTAL = smem_total(OP, CTAS, RB, SPLIT, NC, EW);
    static_assert(SMEM_TOTAL <= SMEM_LIMIT, "shared memory budget");
    // Per kernel variant and device, once: the shared-memory opt-in and (pairs) how many clusters fit the device.
    // Both are properties of the variant, and asking the runtime again on every call costs several microseconds
    // of host time, which is what small problems are bound by.
    static std::atomic<int> ready[64];   // 0 = not set up, else resident blocks / pairs + 1
    int dev = 0;
    int st = rz_record_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (st) return st;
    const bool cacheable = dev >= 0 && dev < 64;
    int known = cacheable ? ready[dev].load(std::memory_order_acquire) : 0;
    if (!known) {
        st = rz_record_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL),
                            "set max dynamic shared memory");
        if (st) return st;
    }

    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    cfg.blockDim = dim3(NTHREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_TOTAL;
    cfg.stream = c.stream;
    cfg.numAttrs = 0;
    // number of blocks (CTAS = 1) or CTA pairs (CTAS = 2) that can be resident at once
    int slots = num_sms() / CTAS;
    if (CTAS == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cfg.gridDim = dim3(2 * (unsigned)slots, 1, 1);
        if (known) {
            slots = known - 1;
        } else {
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) == cudaSuccess && clusters > 0 && clusters < slots)
                slots = clusters;
            (void)cudaGetLastError();
        }
    }
    if (!known && cacheable) ready[dev].store(slots + 1, std::memory_order_release);
    if (pb->sm_reserve > 0) {   // leave SMs idle for whatever the caller runs beside this kernel
        slots -= (pb->sm_reserve + CTAS - 1) / CTAS;
        if (slots < 1) slots = 1;
    }

    const uint32_t tiles = p.tiles_r * p.tiles_c;
    p.nsplit = plan.nsplit > 1 ? (uint32_t)plan.nsplit : 1u;
    p.n_main = plan.nsplit > 1 ? (uint32_t)plan.n_main : tiles;
    if (OP != OP_DW && !p.ws) p.nsplit = 1, p.n_main = tiles;   // no workspace given: whole contraction per block
    if (p.n_main > tiles) p.n_main = tiles;
    if (p.nsplit > p.nchunks) p.nsplit = p.nchunks;
    p.chunks_per_split = (p.nchunks + p.nsplit - 1) / p.nsplit;
    p.nsplit = (p.nchunks + p.chunks_per_split - 1) / p.chunks_per_split;
    if (p.nsplit <= 1) p.nsplit = 1, p.n_main = tiles;
    p.total_items = p.n_main + (tiles - p.n_main) * p.nsplit;
    p.alpha = pb->alpha;
    p.relu = (pb->flags & RZ_FLAG_RELU) ? 1 : 0;
    st = rz_wait_context(&p.wait, 2000000000ll);   // also refuses to launch behind a kernel whose wait gave up
    if (st) return st;
    p.tma_store = knobs().tma_store.load(std::memory_order_relaxed);

    // shared-memory descriptors (bytes)
    const uint32_t atom = KC * 128;
    const uint32_t mn_kstep = (TF32 ? 8 : 16) * 128;  // contraction rows per MMA x 128-byte rows
    const uint32_t mn_sbo = TF32 ? 512 : 1024;        // tf32 M/N-major: rows group by 4 (32-byte-chunk swizzle)
    const uint32_t mn_layout = TF32 ? 1 : 2;
    p.a_layout = p.b_layout = 2;
    if (OP == OP_FWD) {
        p.a_lbo = 16, p.a_sbo = 1024, p.a_kstep = 32;             // K-major
        p.b_lbo = atom, p.b_sbo = mn_sbo, p.b_kstep = mn_kstep;   // N-major
        p.b_layout = mn_layout;
    } else if (OP == OP_DX) {
        p.a_lbo = 16, p.a_sbo = 1024, p.a_kstep = 32;
        p.b_lbo = 16, p.b_sbo = 1024, p.b_kstep = 32;
    } else {
        p.a_lbo = atom, p.a_sbo = mn_sbo, p.a_kstep = mn_kstep;
        p.b_lbo = atom, p.b_sbo = mn_sbo, p.b_kstep = mn_kstep;
        p.a_layout = p.b_layout = mn_layout;
    }
    const uint32_t a_major = (OP == OP_DW) ? 1u : 0u, b_major = (OP == OP_DX) ? 0u : 1u;
    const uint32_t fmt = TF32 ? 2u : 1u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (a_major << 15) | (b_major << 16) | ((uint32_t)(NC >> 3) << 17) |
              ((uint32_t)(PAIR_R >> 4) << 24);

    uint32_t blocks = p.total_items < (uint32_t)slots ? p.total_items : (uint32_t)slots;
    // Small grids whose every block is split anyway (FWD / DX): deal the (block, stage) units out in equal ranges
    // instead of nsplit equal parts per block, so that every SM works whatever the number of blocks (40 blocks in
    // 3 parts keep 120 of 148 SMs busy; 148 ranges keep them all).  Not for split precision, whose parts also
    // bound the accumulation chains.
    p.units = 0;
    if (OP != OP_DW && !SPLIT && p.nsplit > 1 && p.n_main == 0 && knobs().unit_ranges.load(std::memory_order_relaxed)) {
        const uint32_t units = tiles * p.nchunks;
        uint32_t ranges = units / 8 < (uint32_t)slots ? units / 8 : (uint32_t)slots;   // at least 8 stages per range
        if (ranges > blocks) {
            p.units = units;
            blocks = ranges;
        }
    }
    if (knobs().verbose.load(std::memory_order_relaxed))   // bring-up aid: one line per launch on stderr
        fprintf(stderr, "rz_tc op %d tf32 %d block (%d,%d,%d) ew %d stages %d: %u blocks, %u whole + %u x %u parts, %d slots, %u units in %u ranges\n", OP,
                (int)TF32, CTAS, RB, NC, EW, STAGES_HOST, tiles, p.n_main, tiles - p.n_main, p.nsplit, slots, p.units, p.units ? blocks : 0u);
    cfg.gridDim = dim3(blocks * CTAS, 1, 1);
    const bool partial = OP != OP_DW && p.nsplit > 1;
    const uint32_t split_tiles = tiles - p.n_main;
    if (partial) {
        st = rz_record_cuda(cudaMemsetAsync(p.ws, 0, sizeof(float) * (size_t)split_tiles * ITEM_R * NC, c.stream),
                            "zero workspace");
        if (st) return st;
    }
    st = rz_record_cuda(cudaLaunchKernelEx(&cfg, kern, mapA, mapB, mapC, p), "tcgen05 kernel launch");
    rz_count_launch(1);
    if (st) return st;
    st = rz_record_cuda(cudaGetLastError(), "tcgen05 kernel launch");
    if (st || !partial) return st;
    FinalizeGeom fg;
    fg.rows = p.rows, fg.cols = p.cols, fg.item_r = ITEM_R, fg.nc = NC, fg.tiles_r = p.tiles_r, fg.tiles_c = p.tiles_c;
    fg.group_rows = p.group_rows, fg.n_main = p.n_main, fg.n_tiles = tiles;
    // about four CTAs per SM in total, several per block when few blocks were split
    unsigned per_tile = (148u * 4u + split_tiles - 1) / split_tiles;
    if (per_tile > 32u) per_tile = 32u;
    const dim3 fblocks(split_tiles < 148u * 4u ? split_tiles : 148u * 4u, per_tile, 1);
    const float *fbias = OP == OP_FWD ? p.bias : nullptr;   // bias and ReLU belong to the forward pass only
    const int frelu = OP == OP_FWD ? p.relu : 0;
    if (TF32)
        rz_finalize_kernel<float><<<fblocks, 256, 0, c.stream>>>(p.ws, (float *)p.out, fbias, fg, p.alpha, frelu);
    else
        rz_finalize_kernel<__nv_bfloat16><<<fblocks, 256, 0, c.stream>>>(p.ws, (__nv_bfloat16 *)p.out, fbias, fg, p.alpha, frelu);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "finalize launch");
}

template <int OP>
int launch_tc_any(const RzLaunchCtx &c, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC, TcParams &p,
                  const TcConfig &cfg)
{
    const int prec = c.pb->precision;
    if (prec == RZ_PREC_FP32) {   // split precision: fp32 operands, three tf32 MMAs per product
        if (cfg.ctas == 2) return launch_tc<OP, true, 2, 1, 1, 256>(c, mapA, mapB, mapC, p, cfg);
        if (cfg.nc == 256) return launch_tc<OP, true, 1, 1, 1, 256>(c, mapA, mapB, mapC, p, cfg);
        if (cfg.nc == 128) return launch_tc<OP, true, 1, 1, 1, 128>(c, mapA, mapB, mapC, p, cfg);
        return launch_tc<OP, true, 1, 1, 1, 64>(c, mapA, mapB, mapC, p, cfg);
    }
    const bool tf32 = prec == RZ_PREC_TF32;
    if (OP == OP_DW && cfg.ew == 4 && cfg.rb == 1) {   // scatter-bound weight gradient: sixteen epilogue warps
        constexpr int W = (OP == OP_DW) ? 4 : 1;       // (keeps the other operations from instantiating the variant)
        if (cfg.ctas == 2)
            return tf32 ? launch_tc<OP, true, 2, 1, 0, 256, W>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 2, 1, 0, 256, W>(c, mapA, mapB, mapC, p, cfg);
        if (cfg.nc == 256)
            return tf32 ? launch_tc<OP, true, 1, 1, 0, 256, W>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 1, 1, 0, 256, W>(c, mapA, mapB, mapC, p, cfg);
        if (cfg.nc == 128)
            return tf32 ? launch_tc<OP, true, 1, 1, 0, 128, W>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 1, 1, 0, 128, W>(c, mapA, mapB, mapC, p, cfg);
        return tf32 ? launch_tc<OP, true, 1, 1, 0, 64, W>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 1, 1, 0, 64, W>(c, mapA, mapB, mapC, p, cfg);
    }
    if (OP == OP_DW && cfg.ctas == 2 && cfg.rb == 2 && cfg.ew == 2) {
        constexpr int W = (OP == OP_DW) ? 2 : 1;
        return tf32 ? launch_tc<OP, true, 2, 2, 0, 256, W>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 2, 2, 0, 256, W>(c, mapA, mapB, mapC, p, cfg);
    }
    if (cfg.ctas == 2 && cfg.rb == 2)
        return tf32 ? launch_tc<OP, true, 2, 2, 0, 256>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 2, 2, 0, 256>(c, mapA, mapB, mapC, p, cfg);
    if (cfg.ctas == 2)
        return tf32 ? launch_tc<OP, true, 2, 1, 0, 256>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 2, 1, 0, 256>(c, mapA, mapB, mapC, p, cfg);
    if (cfg.nc == 256)
        return tf32 ? launch_tc<OP, true, 1, 1, 0, 256>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 1, 1, 0, 256>(c, mapA, mapB, mapC, p, cfg);
    if (cfg.nc == 128)
        return tf32 ? launch_tc<OP, true, 1, 1, 0, 128>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 1, 1, 0, 128>(c, mapA, mapB, mapC, p, cfg);
    return tf32 ? launch_tc<OP, true, 1, 1, 0, 64>(c, mapA, mapB, mapC, p, cfg) : launch_tc<OP, false, 1, 1, 0, 64>(c, mapA, mapB, mapC, p, cfg);
}

// 2-D map over a row-major matrix [rows][cols] of the operand type
int map_matrix(CUtensorMap *map, bool tf32, bool mn_major, const void *base, uint64_t rows, uint64_t cols,
               uint32_t box_cols, uint32_t box_rows)
{
    const int es = tf32 ? 4 : 2;
    uint64_t dims[2] = {cols, rows};
    uint64_t strides[1] = {cols * (uint64_t)es};
    uint32_t box[2] = {box_cols, box_rows};
    return encode(map, tf32, mn_major, const_cast<void *>(base), 2, dims, strides, box);
}

// 3-D map over the shadow: {element of a copy, slice row (stride BN elements), copy}
int map_shadow(CUtensorMap *map, const rz_problem *pb, bool mn_major, const void *shadow, uint32_t box_rows)
{
    const Geometry g = geometry(pb);
    const bool tf32 = pb->precision != RZ_PREC_BF16;
    uint64_t dims[3] = {g.Hc, (uint64_t)pb->BK, (uint64_t)g.ns};
    uint64_t strides[2] = {(uint64_t)pb->BN * g.es, (uint64_t)g.copy_stride};
    uint32_t box[3] = {(uint32_t)g.epr, box_rows, 1};
    return encode(map, tf32, mn_major, const_cast<void *>(shadow), 3, dims, strides, box);
}

}  // namespace

int rz_tc_wait_selftest(long long limit_cycles, cudaStream_t stream)
{
    RzWaitCtx w;
    int st = rz_wait_context(&w, limit_cycles);
    if (st) return st;
    rz_wait_selftest_kernel<<<1, 32, 0, stream>>>(w);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "wait self-test launch");
}

bool rz_tc_supported(const rz_problem *pb, int op)
{
    (void)op;
    const Geometry g = geometry(pb);
    // a 128-byte operand row must lie inside one hash tile along n; along k a pipeline stage (one such row of
    // contraction elements) is made of whole hash tiles or lies inside one, and tiles are multiples of the 32 rows
    // an epilogue warp scatters
    if (pb->BN % g.epr || pb->BK % 32) return false;
    if (pb->BK < g.epr ? (g.epr % pb->BK != 0) : (pb->BK % g.epr != 0)) return false;
    if (pb->BK <= 64 ? (64 % pb->BK != 0) : (pb->BK % 64 != 0)) return false;   // whole B boxes per hash tile (narrowest block)
    if ((pb->K * g.es) % 16 || (pb->N * g.es) % 16) return false;
    if (pb->K < g.epr || pb->N < g.epr) return false;   // at least one full 128-byte row of every operand
    return true;
}

size_t rz_tc_copies_bytes(const rz_problem *pb)
{
    const Geometry g = geometry(pb);
    return g.copy_stride * (size_t)g.ns;
}

size_t rz_tc_shadow_bytes(const rz_problem *pb)
{
    // the shifted copies, then the fp32 workspace of split-contraction launches (forward and input gradient share it)
    const size_t wf = workspace_bytes(pb, RZ_OP_FORWARD), wi = workspace_bytes(pb, RZ_OP_BACKWARD_INPUT);
    return rz_tc_copies_bytes(pb) + (wf > wi ? wf : wi);
}

bool rz_tc_needs_workspace(const rz_problem *pb, int op)
{
    // split precision bounds its accumulation chains by splitting long contractions: that launch cannot do without
    if (pb->precision != RZ_PREC_FP32 || op == RZ_OP_BACKWARD_WEIGHT) return false;
    return (op == RZ_OP_FORWARD ? pb->K : pb->N) > 2048;
}

void rz_tc_reload_env() { load_knobs(); }

// Workspace of a launch inside the caller's scratch: behind the copies, if the scratch is large enough to hold it
// (a scratch that only holds the copies makes the launch run every block's whole contraction instead).
static int workspace_of(const rz_problem *pb, void *shadow, size_t shadow_bytes, int op, float **ws)
{
    *ws = nullptr;
    const size_t need = workspace_bytes(pb, op), copies = rz_tc_copies_bytes(pb);
    if (shadow_bytes < copies) return RZ_ERR_SCRATCH;
    if (need == 0) return RZ_OK;
    if (shadow_bytes >= copies + need)
        *ws = reinterpret_cast<float *>(static_cast<uint8_t *>(shadow) + copies);
    else if (rz_tc_needs_workspace(pb, op))
        return RZ_ERR_SCRATCH;
    return RZ_OK;
}

int rz_tc_shadow_refresh(const RzLaunchCtx &c, const float *hashed, void *shadow)
{
    const Geometry g = geometry(c.pb);
    const uint32_t groups = g.Hc / g.ns;
    uint32_t blocks = (groups + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (c.pb->precision != RZ_PREC_BF16)
        rz_shadow_kernel<true><<<blocks, 256, 0, c.stream>>>(hashed, (uint8_t *)shadow, (uint32_t)c.pb->H, g.Hc, g.copy_stride,
                                                            c.pb->precision == RZ_PREC_FP32 ? 1 : 0);
    else
        rz_shadow_kernel<false><<<blocks, 256, 0, c.stream>>>(hashed, (uint8_t *)shadow, (uint32_t)c.pb->H, g.Hc, g.copy_stride, 0);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "shadow refresh launch");
}

int rz_tc_sgd_step(const RzLaunchCtx &c, float *hashed, const float *dH, float *velocity, float lr, float momentum, void *shadow)
{
    const uint32_t H = (uint32_t)c.pb->H;
    if (!shadow) {   // no tensor-core scratch to keep in step: the update alone
        uint32_t blocks = velocity ? (H + 255) / 256 : (H / 4 + 255) / 256;
        if (blocks < 1) blocks = 1;
        if (blocks > 148 * 8) blocks = 148 * 8;
        if (velocity) rz_sgd_momentum_kernel<<<blocks, 256, 0, c.stream>>>(hashed, dH, velocity, lr, momentum, H);
        else rz_sgd_kernel<<<blocks, 256, 0, c.stream>>>(hashed, dH, lr, H);
        rz_count_launch(1);
        return rz_record_cuda(cudaGetLastError(), "sgd launch");
    }
    // update + shadow refresh in one pass; each launch in flight draws its own ticket word
    static std::atomic<unsigned> next_ticket{0};
    const unsigned slot = next_ticket.fetch_add(1, std::memory_order_relaxed) % SGD_TICKETS;
    unsigned *ticket = nullptr;
    int st = rz_record_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(&ticket), g_sgd_ticket), "ticket address");
    if (st) return st;
    ticket += slot;
    const Geometry g = geometry(c.pb);
    const uint32_t groups = g.Hc / g.ns;
    uint32_t blocks = (groups + SGD_CHUNK - 1) / SGD_CHUNK;
    if (blocks > 148 * 2) blocks = 148 * 2;
    const bool tf32 = c.pb->precision != RZ_PREC_BF16;
    const int raw = c.pb->precision == RZ_PREC_FP32 ? 1 : 0;
    uint8_t *sh = static_cast<uint8_t *>(shadow);
    if (tf32 && velocity)
        rz_sgd_shadow_kernel<true, true><<<blocks, SGD_CHUNK, 0, c.stream>>>(hashed, dH, velocity, lr, momentum, sh, H, g.Hc, g.copy_stride, raw, ticket);
    else if (tf32)
        rz_sgd_shadow_kernel<true, false><<<blocks, SGD_CHUNK, 0, c.stream>>>(hashed, dH, nullptr, lr, 0.f, sh, H, g.Hc, g.copy_stride, raw, ticket);
    else if (velocity)
        rz_sgd_shadow_kernel<false, true><<<blocks, SGD_CHUNK, 0, c.stream>>>(hashed, dH, velocity, lr, momentum, sh, H, g.Hc, g.copy_stride, 0, ticket);
    else
        rz_sgd_shadow_kernel<false, false><<<blocks, SGD_CHUNK, 0, c.stream>>>(hashed, dH, nullptr, lr, 0.f, sh, H, g.Hc, g.copy_stride, 0, ticket);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "sgd + shadow launch");
}

int rz_tc_forward(const RzLaunchCtx &c, const void *X, void *shadow, size_t shadow_bytes, const float *bias, void *Y)
{
    const rz_problem *pb = c.pb;
    const bool tf32 = pb->precision != RZ_PREC_BF16;
    const Geometry g = geometry(pb);
    TcParams p;
    memset(&p, 0, sizeof(p));
    p.bias = bias;
    p.out = Y;
    int st = workspace_of(pb, shadow, shadow_bytes, RZ_OP_FORWARD, &p.ws);
    if (st) return st;
    CUtensorMap mapA, mapB;
    st = map_matrix(&mapA, tf32, false, X, pb->M, pb->K, g.epr, TILE_R);
    if (st) return st;
    st = map_shadow(&mapB, pb, true, shadow, fwd_box_rows(pb));
    if (st) return st;
    // output map for the epilogue's bulk stores: 32-row x 128-byte boxes
    CUtensorMap mapC;
    st = map_matrix(&mapC, tf32, false, Y, pb->M, pb->N, g.epr, 32);
    if (st) return st;
    return launch_tc_any<OP_FWD>(c, mapA, mapB, mapC, p, choose_config(pb, RZ_OP_FORWARD));
}

int rz_tc_backward_input(const RzLaunchCtx &c, const void *dY, void *shadow, size_t shadow_bytes, void *dX)
{
    const rz_problem *pb = c.pb;
    const bool tf32 = pb->precision != RZ_PREC_BF16;
    const Geometry g = geometry(pb);
    TcParams p;
    memset(&p, 0, sizeof(p));
    p.out = dX;
    int st = workspace_of(pb, shadow, shadow_bytes, RZ_OP_BACKWARD_INPUT, &p.ws);
    if (st) return st;
    CUtensorMap mapA, mapB;
    st = map_matrix(&mapA, tf32, false, dY, pb->M, pb->N, g.epr, TILE_R);
    if (st) return st;
    const TcConfig config = choose_config(pb, RZ_OP_BACKWARD_INPUT);
    st = map_shadow(&mapB, pb, false, shadow, dx_box_rows(pb, config));
    if (st) return st;
    CUtensorMap mapC;
    st = map_matrix(&mapC, tf32, false, dX, pb->M, pb->K, g.epr, 32);
    if (st) return st;
    return launch_tc_any<OP_DX>(c, mapA, mapB, mapC, p, config);
}

int rz_tc_backward_weight(const RzLaunchCtx &c, const void *X, const void *dY, float *dH)
{
    const rz_problem *pb = c.pb;
    const bool tf32 = pb->precision != RZ_PREC_BF16;
    const Geometry g = geometry(pb);
    CUtensorMap mapA, mapB;   // A = dY (accumulator rows = n), B = X (accumulator columns = k)
    int st = map_matrix(&mapA, tf32, true, dY, pb->M, pb->N, g.epr, g.epr);
    if (st) return st;
    st = map_matrix(&mapB, tf32, true, X, pb->M, pb->K, g.epr, g.epr);
    if (st) return st;
    TcParams p;
    memset(&p, 0, sizeof(p));
    p.dH = dH;
    return launch_tc_any<OP_DW>(c, mapA, mapB, mapA, p, choose_config(pb, RZ_OP_BACKWARD_WEIGHT));   // (no output map)
}
