// gemm_tcgen05.cu - persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = alpha * sum_k A(m,k) * B(n,k)   (+ epilogue)
//
// One CTA per SM walks output tiles of 128 x BN (BN = 128 or 256). Warp 0 feeds a multi-stage
// shared-memory ring with TMA tiled loads (128-byte swizzle); warp 1 issues tcgen05.mma from one
// thread with the fp32 accumulator in tensor memory; warps 2-5 drain the accumulator with
// tcgen05.ld and run the epilogue. Two accumulators live in TMEM so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Either operand may be K-major (the reduction dimension is contiguous in memory) or MN-major
// (the M / N dimension is contiguous), which covers forward (X * W^T), input-gradient (dY * W) and
// weight-gradient (dY^T * X) products without materialising a transpose.
//
// Replaces the one-thread-per-output fp32 GEMMs of the reference
// (src/cuda/cai_gpu_train.cu:40-74) and folds its add_k / zero_k passes
// (src/cuda/cai_kernels.cu:161-164, cai_gpu_train.cu:75-78) into the epilogue.
#include "../comm/fused.h"
#include "../comm/gather.cuh"
#include "../comm/peer.cuh"
#include "../plan/formats.h"
#include "cai_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cai {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kAStageBytes = kBM * kBK * 2;
constexpr int kGemmThreads = 192;

struct GemmParams {
    int M, N, K;
    int a_mn, b_mn;
    int epi;
    float alpha;
    void* C;
    const void* R;
    long long ldc, ldr;
    int tiles_m, tiles_n, group_m;
    int* status;
    // ---- fused collective modes (see the block comment above gemm_bf16_kernel)
    int mode;                        // kGemmPlain / kGemmAllGatherA / kGemmReduceScatter
    int group_kind;                  // communicator kind whose signal region is used
    int n_copy;                      // all-gather: leading CTAs that only move rows
    int rows_per_rank;               // rows of the sharded dimension each member owns
    int m_rot;                       // tile rows are walked starting from this block
    const uint32_t* epoch_base;      // device word refreshed by the host every step
    uint32_t seq;                    // per-op sequence number (fixed in the plan)
    unsigned long long src_off;      // all-gather: arena offset of the local rows on every member
    unsigned long long stage_off;    // reduce-scatter: arena offset of the staging buffer on every member
    __nv_bfloat16* a_full;           // all-gather: local buffer that receives every member's rows
    long long ld_src;
    PeerTable pt;
    // ---- ragged segments (expert slabs of a mixture-of-experts layer): the segmented dimension is
    // cut into slabs of seg_rows rows of which only the first seg_counts[slab] hold data.
    // seg_mode 1: the M dimension is segmented, output tiles that start past a slab's count are skipped.
    // seg_mode 2: the K dimension is segmented (weight gradient), k-blocks past a slab's count are skipped.
    const int* seg_counts;
    int seg_rows;
    int seg_mode;
    // ---- groups (the local experts of a mixture-of-experts layer in one launch): `groups` independent
    // products of the same M x N x K; group g reads A / B at row coordinate + g * grp_a / grp_b of their
    // tensor maps, writes C (and reads R) at row + g * grp_c, and owns grp_seg entries of seg_counts.
    int groups;
    long long grp_a, grp_b, grp_c;
    int grp_seg;
    // ---- kGemmGatherB: B lives in a staging buffer that the leading n_copy CTAs fill from the sharded
    // parameter space (gather.cuh); b_elem_off is the element offset of B inside the staged range.
    GatherJob gat;
    long long b_elem_off;
    long long ldb;
    // ---- optional per-CTA time stamps (globaltimer, ns) for the phase tables of the fused modes: 8 words per CTA,
    // see kStamp*; null in production launches.
    unsigned long long* stamps;
    // all-gather mode: tiles [tail_start, tiles) are shared by ALL CTAs, the copy CTAs included: once a copy CTA has
    // staged its units it joins the GEMM for the tail instead of leaving its SM idle. tail_start == tiles: no tail.
    int tail_start;
};

// The tiles one CTA works on, in order; producer, MMA issuer and epilogue warps walk the same sequence.
// Head: tiles [0, tail_start) striped over the compute CTAs. Tail: tiles [tail_start, tiles) striped over the grid.
struct TileWalk {
    int next_head, head_end, head_stride, next_tail, tail_end, tail_stride;
    __device__ __forceinline__ TileWalk(const GemmParams& p, int num_tiles) {
        const int tail0 = p.tail_start < num_tiles ? p.tail_start : num_tiles;
        const int cta = static_cast<int>(blockIdx.x) - p.n_copy;
        head_stride = static_cast<int>(gridDim.x) - p.n_copy;
        head_end = tail0;
        next_head = cta >= 0 ? cta : tail0;          // a copy CTA has no head tiles
        tail_end = num_tiles;
        tail_stride = static_cast<int>(gridDim.x);
        // in the tail the compute CTAs come first, so that they continue with consecutive tiles
        next_tail = tail0 + (cta >= 0 ? cta : head_stride + static_cast<int>(blockIdx.x));
    }
    __device__ __forceinline__ int next() {
        if (next_head < head_end) {
            const int t = next_head;
            next_head += head_stride;
            return t;
        }
        if (next_tail < tail_end) {
            const int t = next_tail;
            next_tail += tail_stride;
            return t;
        }
        return -1;
    }
};

// words of a CTA's stamp record
constexpr int kStampEntry = 0;        // kernel entry
constexpr int kStampFirstReady = 1;   // first tile's operands may be loaded (all-gather: its rows are staged)
constexpr int kStampFirstAcc = 2;     // first accumulator complete
constexpr int kStampLastEpi = 3;      // last tile's epilogue (and pushes) done
constexpr int kStampReduceStart = 4;  // reduce-scatter: reduce phase entered
constexpr int kStampReduceFlags = 5;  // reduce-scatter: every member's partial of the first item has arrived
constexpr int kStampEnd = 6;          // CTA done
constexpr int kStampCopyDone = 7;     // all-gather copy CTA: last unit staged
__device__ __forceinline__ void stamp(const GemmParams& p, int word) {
    if (p.stamps) p.stamps[static_cast<size_t>(blockIdx.x) * 8 + word] = global_timer_ns();
}

__device__ __forceinline__ bool seg_live(const GemmParams& p, int g, int row0) {
    const int slab = row0 / p.seg_rows;
    return row0 - slab * p.seg_rows < p.seg_counts[g * p.grp_seg + slab];
}

constexpr int kGemmPlain = 0, kGemmAllGatherA = 1, kGemmReduceScatter = 2, kGemmGatherB = 3;

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile_all, int& tm, int& tn, int& grp) {
    const int tiles_per_product = p.tiles_m * p.tiles_n;
    grp = tile_all / tiles_per_product;
    const int tile = tile_all - grp * tiles_per_product;
    const int per_group = p.group_m * p.tiles_n;
    const int g = tile / per_group;
    const int first_m = g * p.group_m;
    const int gsz = min(p.tiles_m - first_m, p.group_m);
    const int in = tile - g * per_group;
    tm = first_m + in % gsz;
    tn = in / gsz;
    if (p.m_rot) {
        tm += p.m_rot;
        if (tm >= p.tiles_m) tm -= p.tiles_m;
    }
}

__device__ __forceinline__ void bar_sync_epilogue() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// All-gather staging, run by the leading CTAs of the grid: one thread per copy CTA drives the TMA
// engine, pulling every member's rows (bulk loads over NVLink, 128 rows per unit) through a ring of
// shared-memory slots into the local gathered buffer, and publishes one local flag per 128-row
// block that the TMA producers of the compute CTAs wait on. Several pieces are in flight per CTA,
// which is what it takes to fill an NVLink.
constexpr int kAgSlots = 6;
constexpr uint32_t kAgPiece = 32768;

__device__ __forceinline__ bool allgather_copy_role(const GemmParams& p, uint32_t epoch, uint8_t* ring, uint64_t* bars) {
    volatile int no_abort = 0;
    for (int i = 0; i < kAgSlots; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
    const int blocks_per_rank = p.rows_per_rank / kBM;
    const int units = p.pt.size * blocks_per_rank;
    const size_t row_bytes = static_cast<size_t>(p.K) * 2;
    const bool contiguous = p.ld_src == p.K;
    // a piece is a contiguous byte range: 32 KiB of a contiguous block, or one row otherwise
    const uint32_t piece = contiguous ? kAgPiece : static_cast<uint32_t>(row_bytes);
    const uint32_t pieces = static_cast<uint32_t>(contiguous ? (kBM * row_bytes) / kAgPiece : kBM);
    uint32_t n = 0;  // pieces issued by this CTA so far (slot = n % kAgSlots, phase = (n / kAgSlots) & 1)
    for (int u = blockIdx.x; u < units; u += p.n_copy) {
        // the peers in ring order, own rows last: the compute CTAs read the own rows from their source, the staged
        // copy only serves later readers of the gathered buffer
        const int s = (p.pt.rank + 1 + u / blocks_per_rank) % p.pt.size;
        const int j = u % blocks_per_rank;
        if (!wait_flag_ge(sig_word(p.pt, p.pt.rank, p.group_kind, kSigEntry + s), epoch, p.status)) return false;
        const uint8_t* src = p.pt.base[s] + p.src_off + static_cast<size_t>(j) * kBM * p.ld_src * 2;
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.a_full) + (static_cast<size_t>(s) * p.rows_per_rank + j * kBM) * row_bytes;
        const size_t src_step = contiguous ? piece : static_cast<size_t>(p.ld_src) * 2;
        constexpr uint32_t kLag = kAgSlots - 2;  // loads in flight ahead of the store
        for (uint32_t i = 0; i < pieces + kLag; ++i) {
            if (i < pieces) {
                const uint32_t slot = n % kAgSlots;
                if (n >= kAgSlots) bulk_wait_read1();  // the store that last used this slot has read it
                mbar_expect_tx(&bars[slot], piece);
                bulk_load(ring + slot * kAgPiece, src + i * src_step, piece, &bars[slot]);
                ++n;
            }
            if (i >= kLag) {
                const uint32_t m = n - (i < pieces ? kLag + 1 : pieces + kLag - i);  // global index of the piece to store
                const uint32_t slot = m % kAgSlots;
                if (!mbar_wait(&bars[slot], (m / kAgSlots) & 1, &no_abort, p.status, CAI_DEV_TIMEOUT_TMA_FULL)) return false;
                bulk_store(dst + static_cast<size_t>(i - kLag) * piece, ring + slot * kAgPiece, piece);
                tma_store_commit();
            }
        }
        tma_store_wait0();
        fence_proxy_async_all();
        __threadfence();
        uint32_t* flag = sig_word(p.pt, p.pt.rank, p.group_kind, kSigLocal + s * blocks_per_rank + j);
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
    }
    return true;
}

// Reduce-scatter epilogue staging: 128 columns at a time (32 rows x (256 + 16) bytes per epilogue warp), which
// leaves room for a fourth operand stage. The kernel has no static shared memory, so the dynamic window starts
// 1 KB aligned and needs no alignment slack in practice; the reduce-scatter variant budgets 768 bytes.
constexpr int kRsCols = 128;
constexpr int kRsPitch = kRsCols * 2 + 16;
constexpr int kRsStageBytes = 4 * 32 * kRsPitch;
template <bool RS>
__host__ __device__ constexpr int gemm_align_slack() { return RS ? 768 : 1024; }

template <int BN, int STAGES, bool RS>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const GemmParams p) {
    // tmA2: all-gather mode only, this member's own rows where they were produced (no staging, no wait)
    constexpr int kBStageBytes = BN * kBK * 2;
    constexpr int kStageBytes = kAStageBytes + kBStageBytes;
    constexpr uint32_t kTmemCols = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    if (static_cast<int>(smem - smem_raw) > gemm_align_slack<RS>()) {
        // the launch reserved less slack than this base address needs: report instead of running past the end
        if (threadIdx.x == 0) atomicCAS(p.status, 0, CAI_DEV_BAD_ARG);
        return;
    }
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * kAStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tmem_full = bars + 2 * STAGES;
    uint64_t* tmem_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Fused modes. kGemmAllGatherA: A is the row-wise concatenation of every member's local rows;
    // the first n_copy CTAs pull them into a_full and the TMA producers wait per 128-row block.
    // kGemmReduceScatter: the epilogue pushes each bf16 tile into the staging buffer of the member
    // that owns those rows (peer stores) and raises a per-tile flag there; when a CTA has no GEMM
    // tiles left it sums, for output tiles of its own rows, the partials of all members (+ residual).
    uint32_t epoch = 0;
    if (threadIdx.x == 0) stamp(p, kStampEntry);
    if (p.mode != kGemmPlain) {
        epoch = *p.epoch_base + 2 * p.seq;
        if (p.mode == kGemmAllGatherA) {
            if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(p.pt, p.group_kind, kSigEntry + p.pt.rank, epoch);
            if (static_cast<int>(blockIdx.x) < p.n_copy) {
                // the ring's barriers sit behind the GEMM pipeline's (which this CTA initialises afterwards if it joins)
                volatile int* copy_ok = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(bars) + 196);
                if (threadIdx.x == 0) {
                    *copy_ok = allgather_copy_role(p, epoch, smem, reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(bars) + 200)) ? 1 : 0;
                    stamp(p, kStampCopyDone);
                }
                __syncthreads();
                if (!*copy_ok || p.tail_start >= p.tiles_m * p.tiles_n * p.groups) return;
            }
        }
        if (p.mode == kGemmGatherB && static_cast<int>(blockIdx.x) < p.n_copy) {
            // parameter shards are stable for the whole forward / backward pass: no entry handshake
            if (threadIdx.x == 0) gather_copy_role(p.pt, p.gat, static_cast<int>(blockIdx.x), epoch, smem, bars, p.status);
            return;
        }
    }
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.tiles_m * p.tiles_n * p.groups;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            TileWalk walk(p, num_tiles);
            bool first_tile = true;
            for (int tile = walk.next(); tile >= 0 && ok; tile = walk.next()) {
                int tm, tn, grp;
                tile_coords(p, tile, tm, tn, grp);
                const int m0 = tm * kBM, n0 = tn * BN;
                if (p.seg_mode == 1 && !seg_live(p, grp, m0)) continue;
                const int ga = static_cast<int>(grp * p.grp_a), gb = static_cast<int>(grp * p.grp_b);
                const int own_blk0 = p.mode == kGemmAllGatherA ? p.pt.rank * (p.rows_per_rank / kBM) : 0;
                const bool local_rows = p.mode == kGemmAllGatherA && tm >= own_blk0 && tm < own_blk0 + p.rows_per_rank / kBM;
                if (p.mode == kGemmAllGatherA && !local_rows) {
                    // rows of this tile must have been staged by a copy CTA; they were written through
                    // the generic proxy, the TMA engine reads through the async proxy
                    const uint32_t* flag = sig_word(p.pt, p.pt.rank, p.group_kind, kSigLocal + tm);
                    bool seen = false, timed_out = false;
                    // the copy CTA that raises this flag waits on a peer itself: its whole limit and a little more
                    const uint64_t t0 = global_timer_ns(), limit = peer_wait_limit_ns(p.status) * 5 / 4;
                    for (uint32_t it = 0; !seen; ++it) {
                        uint32_t v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                        seen = static_cast<int32_t>(v - epoch) >= 0;
                        if (!seen && !peer_spin_continue(it, t0, limit, p.status, &timed_out)) break;
                    }
                    if (!seen) {
                        *abort_flag = 1;
                        if (timed_out) atomicCAS(p.status, 0, CAI_DEV_TIMEOUT_PEER_FLAG);
                        ok = false;
                        break;
                    }
                    fence_proxy_async_all();
                }
                if (p.mode == kGemmGatherB) {
                    // the rows of B this tile reads must have been staged by a copy CTA
                    long long x = p.b_elem_off, y;
                    if (!p.b_mn) {
                        const int n1 = n0 + BN < p.N ? n0 + BN : p.N;
                        y = x + static_cast<long long>(n1) * p.ldb;
                        x += static_cast<long long>(n0) * p.ldb;
                    } else {
                        y = x + static_cast<long long>(p.K) * p.ldb;
                    }
                    if (!gather_wait_range(p.pt, p.gat, x, y, epoch, p.status)) {
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                }
                if (first_tile) stamp(p, kStampFirstReady);
                first_tile = false;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (p.seg_mode == 2 && !seg_live(p, grp, kb * kBK)) continue;
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMA_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], kStageBytes);
                    uint8_t* a_dst = sA + s * kAStageBytes;
                    uint8_t* b_dst = sB + s * kBStageBytes;
                    const int k0 = kb * kBK;
                    if (local_rows) {
                        tma_load_2d(a_dst, &tmA2, &full[s], k0, m0 - own_blk0 * kBM);   // my rows, straight from their source
                    } else if (!p.a_mn) {
                        tma_load_2d(a_dst, &tmA, &full[s], k0, m0 + ga);
                    } else {
#pragma unroll
                        for (int c = 0; c < kBM / 64; ++c)
                            tma_load_2d(a_dst + c * (kBK * 128), &tmA, &full[s], m0 + c * 64, k0 + ga);
                    }
                    if (p.epi == CAI_EPI_SWIGLU) {
                        // gate rows and the up rows of the same features, stacked in one stage
                        const int F = p.N >> 1, j0 = tn * (BN / 2);
                        tma_load_2d(b_dst, &tmB, &full[s], k0, j0 + gb);
                        tma_load_2d(b_dst + (BN / 2) * kBK * 2, &tmB, &full[s], k0, F + j0 + gb);
                    } else if (!p.b_mn) {
                        tma_load_2d(b_dst, &tmB, &full[s], k0, n0 + gb);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tma_load_2d(b_dst + c * (kBK * 128), &tmB, &full[s], n0 + c * 64, k0 + gb);
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok) {
                // Give copies still in flight time to land before the CTA's memory is released.
                for (int i = 0; i < 32; ++i) __nanosleep(50000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer
            const uint32_t idesc = umma_idesc_bf16(kBM, BN, p.a_mn, p.b_mn);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int t = 0;
            TileWalk walk(p, num_tiles);
            for (int tile = walk.next(); tile >= 0 && ok; tile = walk.next()) {
                int grp = 0;
                if (p.seg_mode) {
                    int tm, tn;
                    tile_coords(p, tile, tm, tn, grp);
                    if (p.seg_mode == 1 && !seg_live(p, grp, tm * kBM)) continue;
                }
                const int acc = t & 1;
                const uint32_t acc_ph = (t >> 1) & 1;
                ++t;
                if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMEM_EMPTY)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                uint32_t started = 0;  // becomes 1 after the first MMA of the tile (which overwrites the accumulator)
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (p.seg_mode == 2 && !seg_live(p, grp, kb * kBK)) continue;
                    if (!mbar_wait(&full[s], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_TMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(sA + s * kAStageBytes);
                    const uint32_t b_base = smem_u32(sB + s * kBStageBytes);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        const uint64_t adesc =
                            p.a_mn ? umma_smem_desc_sw128(a_base + k * (kUmmaK * 128), kBK * 128, 1024)
                                   : umma_smem_desc_sw128(a_base + k * (kUmmaK * 2), 0, 1024);
                        const uint64_t bdesc =
                            p.b_mn ? umma_smem_desc_sw128(b_base + k * (kUmmaK * 128), kBK * 128, 1024)
                                   : umma_smem_desc_sw128(b_base + k * (kUmmaK * 2), 0, 1024);
                        umma_f16_ss(d_tmem, adesc, bdesc, idesc, started);
                        started = 1;
                    }
                    umma_commit(&empty[s]);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(&tmem_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue warps: TMEM -> registers -> global
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int t = 0;
        bool ok = true;
        int rs_prev_owner = -1;
        uint32_t rs_prev_slot = 0;
        bool rs_reduce_seen = false;
        (void)rs_prev_owner; (void)rs_prev_slot; (void)rs_reduce_seen;
        TileWalk walk(p, num_tiles);
        for (int tile = walk.next(); tile >= 0 && ok; tile = walk.next()) {
            int tm, tn, grp;
            tile_coords(p, tile, tm, tn, grp);
            if (p.seg_mode == 1 && !seg_live(p, grp, tm * kBM)) continue;
            const int acc = t & 1;
            const uint32_t acc_ph = (t >> 1) & 1;
            ++t;
            // a weight-gradient tile whose every k-block was skipped has an undefined accumulator: it counts as zero
            bool acc_valid = true;
            if (p.seg_mode == 2) {
                acc_valid = false;
                for (int kb = 0; kb < num_kb && !acc_valid; ++kb) acc_valid = seg_live(p, grp, kb * kBK);
            }
            if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.status, CAI_DEV_TIMEOUT_TMEM_FULL)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (t == 1 && warp == 2 && lane == 0) stamp(p, kStampFirstAcc);
            if constexpr (RS) {
                // Reduce-scatter epilogue: the warp's 32 rows x BN bf16 are staged in shared memory
                // and every lane hands its row (one contiguous run in the owner's staging buffer) to
                // the TMA engine as a bulk store over NVLink. The tile's arrival flag is raised one
                // tile late, once the stores of that tile have completed, so that the wait for remote
                // completion overlaps the next tile.
                uint8_t* stg = smem + STAGES * kStageBytes + 256 + q * 32 * kRsPitch;
                const long long row = (long long)tm * kBM + q * 32 + lane;
                const int blocks_per_rank = p.rows_per_rank / kBM;
                const int owner = tm / blocks_per_rank;
                const long long lrow = row - static_cast<long long>(owner) * p.rows_per_rank;
                __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.pt.base[owner] + p.stage_off) +
                                      (static_cast<long long>(p.pt.rank) * p.rows_per_rank + lrow) * p.N + tn * BN;
                const float alpha = p.alpha;
                if (owner == p.pt.rank) {
                    // A tile of MY rows (they come last in the walk): nothing is pushed. The other members sent their
                    // partials of these rows early (each walks its own rows last too), so the reduction happens right
                    // here: accumulator (still fp32) + every member's partial from my staging buffer + residual ->
                    // the final rows. No separate reduce pass trails the GEMM.
                    volatile int* rs_ok = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(bars) + 192);
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // pushes of the tile before this one
                    fence_proxy_async_all();
                    bar_sync_epilogue();
                    if (warp == 2 && lane == 0) {
                        if (rs_prev_owner >= 0) {
                            __threadfence_system();
                            st_release_sys(sig_word(p.pt, rs_prev_owner, p.group_kind, kSigTile + p.pt.rank * kSigTileSlots + rs_prev_slot), epoch);
                        }
                        if (!rs_reduce_seen) stamp(p, kStampReduceStart);
                        const uint32_t item = static_cast<uint32_t>((tm - owner * blocks_per_rank) * p.tiles_n + tn);
                        int good = 1;
                        for (int src = 0; src < p.pt.size && good; ++src)
                            if (src != p.pt.rank)
                                good = wait_flag_ge(sig_word(p.pt, p.pt.rank, p.group_kind, kSigTile + src * kSigTileSlots + item), epoch,
                                                    p.status) ? 1 : 0;
                        *rs_ok = good;
                        if (!rs_reduce_seen) stamp(p, kStampReduceFlags);
                    }
                    rs_reduce_seen = true;
                    rs_prev_owner = -1;
                    bar_sync_epilogue();
                    if (!*rs_ok) {
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(p.pt.base[p.pt.rank] + p.stage_off);
                    const bool row_ok = lrow < p.rows_per_rank;
#pragma unroll 1
                    for (int c = 0; c < BN / 32; ++c) {
                        uint32_t r[32];
                        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32;
                        tmem_ld_32x32(taddr, r);
                        tmem_ld_wait();
                        const int col0 = tn * BN + c * 32;
                        if (!row_ok || col0 >= p.N) continue;
                        float v[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]) * alpha;
                        const int nv = (p.N - col0) >= 32 ? 4 : (p.N - col0) / 8;   // 16-byte vectors of this chunk inside N
                        // every member's partial of 16 columns is requested before the first one is consumed: the loop
                        // is bound by the latency of these loads, so as many as the registers allow are in flight
#pragma unroll
                        for (int hv = 0; hv < 2; ++hv) {
                            uint4 pv[kMaxPeers][2];
#pragma unroll
                            for (int src = 0; src < kMaxPeers; ++src) {
                                if (src < p.pt.size && src != p.pt.rank) {
                                    const uint4* prow = reinterpret_cast<const uint4*>(
                                        stage + (static_cast<long long>(src) * p.rows_per_rank + lrow) * p.N + col0);
                                    if (hv * 2 < nv) pv[src][0] = prow[hv * 2];
                                    if (hv * 2 + 1 < nv) pv[src][1] = prow[hv * 2 + 1];
                                }
                            }
#pragma unroll
                            for (int src = 0; src < kMaxPeers; ++src) {
                                if (src < p.pt.size && src != p.pt.rank) {
#pragma unroll
                                    for (int k = 0; k < 2; ++k) {
                                        const int j = hv * 2 + k;
                                        if (j < nv) {
                                            v[j * 8 + 0] += bf16_lo(pv[src][k].x); v[j * 8 + 1] += bf16_hi(pv[src][k].x);
                                            v[j * 8 + 2] += bf16_lo(pv[src][k].y); v[j * 8 + 3] += bf16_hi(pv[src][k].y);
                                            v[j * 8 + 4] += bf16_lo(pv[src][k].z); v[j * 8 + 5] += bf16_hi(pv[src][k].z);
                                            v[j * 8 + 6] += bf16_lo(pv[src][k].w); v[j * 8 + 7] += bf16_hi(pv[src][k].w);
                                        }
                                    }
                                }
                            }
                        }
                        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + lrow * p.ldc + col0;
                        const uint4* rrow = p.R ? reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.R) + lrow * p.ldr + col0) : nullptr;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (j >= nv) break;
                            if (rrow) {
                                const uint4 rv = rrow[j];
                                v[j * 8 + 0] += bf16_lo(rv.x); v[j * 8 + 1] += bf16_hi(rv.x);
                                v[j * 8 + 2] += bf16_lo(rv.y); v[j * 8 + 3] += bf16_hi(rv.y);
                                v[j * 8 + 4] += bf16_lo(rv.z); v[j * 8 + 5] += bf16_hi(rv.z);
                                v[j * 8 + 6] += bf16_lo(rv.w); v[j * 8 + 7] += bf16_hi(rv.w);
                            }
                            uint4 o;
                            o.x = pack_bf16(v[j * 8 + 0], v[j * 8 + 1]); o.y = pack_bf16(v[j * 8 + 2], v[j * 8 + 3]);
                            o.z = pack_bf16(v[j * 8 + 4], v[j * 8 + 5]); o.w = pack_bf16(v[j * 8 + 6], v[j * 8 + 7]);
                            *reinterpret_cast<uint4*>(crow + j * 8) = o;
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[acc]);
                    continue;
                }
#pragma unroll 1
                for (int h = 0; h < BN / kRsCols; ++h) {
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staging free again
                    __syncwarp();
#pragma unroll 1
                    for (int c = 0; c < kRsCols / 32; ++c) {
                        uint32_t r[32];
                        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + h * kRsCols + c * 32;
                        tmem_ld_32x32(taddr, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 o;
                            o.x = pack_bf16(__uint_as_float(r[j * 8 + 0]) * alpha, __uint_as_float(r[j * 8 + 1]) * alpha);
                            o.y = pack_bf16(__uint_as_float(r[j * 8 + 2]) * alpha, __uint_as_float(r[j * 8 + 3]) * alpha);
                            o.z = pack_bf16(__uint_as_float(r[j * 8 + 4]) * alpha, __uint_as_float(r[j * 8 + 5]) * alpha);
                            o.w = pack_bf16(__uint_as_float(r[j * 8 + 6]) * alpha, __uint_as_float(r[j * 8 + 7]) * alpha);
                            *reinterpret_cast<uint4*>(stg + lane * kRsPitch + c * 64 + j * 16) = o;
                        }
                    }
                    const bool last_half = h == BN / kRsCols - 1;
                    if (last_half) tc_fence_before();
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (last_half && lane == 0) mbar_arrive(&tmem_empty[acc]);
                    const int left = p.N - (tn * BN + h * kRsCols);
                    const int cols = left < kRsCols ? left : kRsCols;
                    if (cols > 0) bulk_store(drow + h * kRsCols, stg + lane * kRsPitch, static_cast<uint32_t>(cols) * 2);
                    tma_store_commit();   // one (possibly empty) group per half
                }
                // announce the previous tile: its stores (all but this tile's groups) have completed
                if constexpr (BN / kRsCols == 2) asm volatile("cp.async.bulk.wait_group 2;" ::: "memory");
                else asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
                fence_proxy_async_all();
                bar_sync_epilogue();   // every lane's stores of the previous tile have completed
                if (warp == 2 && lane == 0 && rs_prev_owner >= 0) {
                    // one system-scope fence by the signalling thread (cumulative over what the barrier ordered)
                    __threadfence_system();
                    st_release_sys(sig_word(p.pt, rs_prev_owner, p.group_kind, kSigTile + p.pt.rank * kSigTileSlots + rs_prev_slot), epoch);
                }
                rs_prev_owner = owner;
                rs_prev_slot = static_cast<uint32_t>((tm - owner * blocks_per_rank) * p.tiles_n + tn);
            } else {
            const long long row_in = (long long)tm * kBM + q * 32 + lane;   // row inside this group's product
            const bool row_ok = row_in < p.M;
            const long long row = row_in + grp * p.grp_c;
            if (p.epi == CAI_EPI_SWIGLU) {
                // accumulator columns [0, BN/2) are gate, [BN/2, BN) up, of features j0 .. j0 + BN/2
                const int F = p.N >> 1, j0 = tn * (BN / 2);
                __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc;
                __nv_bfloat16* arow = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p.R)) + row * p.ldr;
#pragma unroll 1
                for (int c = 0; c < BN / 64; ++c) {
                    uint32_t rg[32], ru[32];
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32;
                    tmem_ld_32x32(taddr, rg);
                    tmem_ld_32x32(taddr + BN / 2, ru);
                    tmem_ld_wait();
                    const int j = j0 + c * 32;
                    if (!row_ok || j >= F) continue;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        if (j + v * 8 >= F) break;
                        uint4 og, ou, oa;
                        uint32_t* pg = &og.x; uint32_t* pu = &ou.x; uint32_t* pa = &oa.x;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // round to bf16 first: the activation is computed from the values the backward will read
                            pg[e] = pack_bf16(__uint_as_float(rg[v * 8 + 2 * e]) * p.alpha, __uint_as_float(rg[v * 8 + 2 * e + 1]) * p.alpha);
                            pu[e] = pack_bf16(__uint_as_float(ru[v * 8 + 2 * e]) * p.alpha, __uint_as_float(ru[v * 8 + 2 * e + 1]) * p.alpha);
                            const float g0 = bf16_lo(pg[e]), g1 = bf16_hi(pg[e]), u0 = bf16_lo(pu[e]), u1 = bf16_hi(pu[e]);
                            pa[e] = pack_bf16(g0 * (1.f / (1.f + __expf(-g0))) * u0, g1 * (1.f / (1.f + __expf(-g1))) * u1);
                        }
                        *reinterpret_cast<uint4*>(crow + j + v * 8) = og;
                        *reinterpret_cast<uint4*>(crow + F + j + v * 8) = ou;
                        *reinterpret_cast<uint4*>(arow + j + v * 8) = oa;
                    }
                }
            } else {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32;
                tmem_ld_32x32(taddr, r);
                tmem_ld_wait();
                if (!acc_valid) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) r[e] = 0u;
                }
                const int col0 = tn * BN + c * 32;
                if (!row_ok || col0 >= p.N) continue;
                const float alpha = p.alpha;
                if (p.epi == CAI_EPI_SWIGLU_BWD) {
                    // acc = dact[row, col]; R = saved [gate | up]; C = [dgate | dup]
                    const int F = p.N;
                    const __nv_bfloat16* grow = reinterpret_cast<const __nv_bfloat16*>(p.R) + row * p.ldr + col0;
                    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (col0 + j * 8 >= p.N) break;
                        const uint4 gv = *reinterpret_cast<const uint4*>(grow + j * 8);
                        const uint4 uv = *reinterpret_cast<const uint4*>(grow + F + j * 8);
                        const uint32_t* pg = &gv.x; const uint32_t* pu = &uv.x;
                        uint4 odg, odu;
                        uint32_t* pdg = &odg.x; uint32_t* pdu = &odu.x;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // dact goes through bf16 like the tensor it replaces
                            const uint32_t dd = pack_bf16(__uint_as_float(r[j * 8 + 2 * e]) * alpha, __uint_as_float(r[j * 8 + 2 * e + 1]) * alpha);
                            const float d0 = bf16_lo(dd), d1 = bf16_hi(dd);
                            const float g0 = bf16_lo(pg[e]), g1 = bf16_hi(pg[e]), u0 = bf16_lo(pu[e]), u1 = bf16_hi(pu[e]);
                            const float s0 = 1.f / (1.f + __expf(-g0)), s1 = 1.f / (1.f + __expf(-g1));
                            pdg[e] = pack_bf16(d0 * u0 * s0 * (1.f + g0 * (1.f - s0)), d1 * u1 * s1 * (1.f + g1 * (1.f - s1)));
                            pdu[e] = pack_bf16(d0 * (g0 * s0), d1 * (g1 * s1));
                        }
                        *reinterpret_cast<uint4*>(orow + j * 8) = odg;
                        *reinterpret_cast<uint4*>(orow + F + j * 8) = odu;
                    }
                } else if (p.epi == CAI_EPI_BF16 || p.epi == CAI_EPI_BF16_RESIDUAL) {
                    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
                    const __nv_bfloat16* rrow =
                        p.epi == CAI_EPI_BF16_RESIDUAL
                            ? reinterpret_cast<const __nv_bfloat16*>(p.R) + row * p.ldr + col0
                            : nullptr;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (col0 + j * 8 >= p.N) break;
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]) * alpha;
                        if (rrow) {
                            const uint4 rv = *reinterpret_cast<const uint4*>(rrow + j * 8);
                            v[0] += bf16_lo(rv.x); v[1] += bf16_hi(rv.x);
                            v[2] += bf16_lo(rv.y); v[3] += bf16_hi(rv.y);
                            v[4] += bf16_lo(rv.z); v[5] += bf16_hi(rv.z);
                            v[6] += bf16_lo(rv.w); v[7] += bf16_hi(rv.w);
                        }
                        uint4 o;
                        o.x = pack_bf16(v[0], v[1]);
                        o.y = pack_bf16(v[2], v[3]);
                        o.z = pack_bf16(v[4], v[5]);
                        o.w = pack_bf16(v[6], v[7]);
                        *reinterpret_cast<uint4*>(crow + j * 8) = o;
                    }
                } else {
                    float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
                    const bool accum = p.epi == CAI_EPI_F32_ACCUM;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (col0 + j * 4 >= p.N) break;
                        float4 o;
                        o.x = __uint_as_float(r[j * 4 + 0]) * alpha;
                        o.y = __uint_as_float(r[j * 4 + 1]) * alpha;
                        o.z = __uint_as_float(r[j * 4 + 2]) * alpha;
                        o.w = __uint_as_float(r[j * 4 + 3]) * alpha;
                        if (accum) {
                            const float4 old = *reinterpret_cast<const float4*>(crow + j * 4);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        *reinterpret_cast<float4*>(crow + j * 4) = o;
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
            }
        }
        if constexpr (!RS) {
            if (warp == 2 && lane == 0) stamp(p, kStampLastEpi);
        }
        if constexpr (RS) {
            // the last tile's stores: wait for completion, then announce it
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            fence_proxy_async_all();
            bar_sync_epilogue();
            if (warp == 2 && lane == 0 && rs_prev_owner >= 0) {
                __threadfence_system();
                st_release_sys(sig_word(p.pt, rs_prev_owner, p.group_kind, kSigTile + p.pt.rank * kSigTileSlots + rs_prev_slot), epoch);
            }
            if (warp == 2 && lane == 0) stamp(p, kStampLastEpi);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) stamp(p, kStampEnd);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int BN, int STAGES, bool RS>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2, GemmParams& p, int sms,
                       cudaStream_t stream) {
    constexpr int smem_bytes = STAGES * (kAStageBytes + BN * kBK * 2) + gemm_align_slack<RS>() + 256 + (RS ? kRsStageBytes : 0);
    static_assert(smem_bytes <= 232448, "shared memory per CTA");
    static bool configured[64] = {};
    const int dev = current_device();
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes) != cudaSuccess) {
            set_last_error("cudaFuncSetAttribute(gemm) failed: %s", cudaGetErrorString(cudaGetLastError()));
            return CAI_K_CUDA;
        }
        configured[dev & 63] = true;
    }
    p.tiles_m = (p.M + kBM - 1) / kBM;
    p.tiles_n = (p.N + BN - 1) / BN;
    // gather mode walks every row block of an output column before the next column, so that the columns of B
    // are needed in the order the copy CTAs stage them (A stays L2 resident)
    p.group_m = p.mode == kGemmGatherB ? p.tiles_m : 8;
    const int tiles = p.tiles_m * p.tiles_n * p.groups;
    int grid = tiles < sms - p.n_copy ? tiles : sms - p.n_copy;
    if (grid < 1) grid = 1;
    grid += p.n_copy;
    if (p.mode == kGemmReduceScatter && (p.rows_per_rank / kBM) * p.tiles_n > static_cast<int>(kSigTileSlots)) {
        set_last_error("gemm_rs: too many tiles per member for the signal block");
        return CAI_K_BAD_ARG;
    }
    if (p.mode == kGemmAllGatherA && p.n_copy > 0) {
        // the last quarter of the tiles is shared with the copy CTAs, which have staged their units by then
        // The head lasts about as long as the copy: one copy CTA moves ~45 GB/s through its shared-memory ring, one
        // compute CTA finishes a 128 x BN x K tile at ~8.4 TFLOP/s. What is left after that many waves is the tail.
        const int ncomp = grid - p.n_copy;
        const double copy_us = static_cast<double>(p.M) * p.K * 2.0 / p.n_copy / 45e3;
        const double tile_us = 2.0 * kBM * BN * static_cast<double>(p.K) / 8.4e6;
        const long long head = static_cast<long long>(copy_us / tile_us + 1.0) * ncomp;
        p.tail_start = head < tiles ? static_cast<int>(head) : tiles;
    }
    gemm_bf16_kernel<BN, STAGES, RS><<<grid, kGemmThreads, smem_bytes, stream>>>(tmA, tmB, tmA2, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("gemm launch failed: %s", cudaGetErrorString(e));
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}

// Debug aid of the micro-benchmarks: when set, the next launches of the fused modes record per-CTA time stamps.
static unsigned long long* g_stamp_buf[64] = {};

// Picks the tile width, encodes the tensor maps and launches. `p` carries everything but the
// tile bookkeeping.
static int gemm_dispatch(const void* A, const void* B, long long lda, long long ldb, GemmParams& p, int sm_limit,
                         cudaStream_t st) {
    const int M = p.M, N = p.N, K = p.K;
    const int dev = current_device();
    int sms = sm_count(dev);
    if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
    const int usable = sms - p.n_copy > 0 ? sms - p.n_copy : 1;
    // Tile width: fewer, wider tiles amortise the A operand better; narrower tiles quantise
    // into waves better when the output is small.
    auto cost = [&](int bn) {
        const long long tiles = (long long)((M + kBM - 1) / kBM) * ((N + bn - 1) / bn) * p.groups;
        const long long waves = (tiles + usable - 1) / usable;
        // a 128-wide tile streams 128 B/clk/SM of operands for half the math of a 256-wide one and runs
        // at the L2 limit: measured 27.6 us against 30 us per wave at K = 4096, i.e. 1.84x the cost per FLOP
        return (double)waves * bn * (bn == 128 ? 1.84 : 1.0);
    };
    const int BN = cost(256) <= cost(128) ? 256 : 128;
    CUtensorMap tmA, tmB;
    bool ok;
    // the maps of a grouped launch span every group's rows
    const long long xa = (p.groups - 1) * p.grp_a, xb = (p.groups - 1) * p.grp_b;
    if (!p.a_mn) ok = encode_tmap_2d(&tmA, A, M + xa, K, lda, kBK, kBM, 2);
    else ok = encode_tmap_2d(&tmA, A, K + xa, M, lda, 64, kBK, 2);
    if (!ok) return CAI_K_BAD_ARG;
    if (p.epi == CAI_EPI_SWIGLU) ok = encode_tmap_2d(&tmB, B, N + xb, K, ldb, kBK, BN / 2, 2);
    else if (!p.b_mn) ok = encode_tmap_2d(&tmB, B, N + xb, K, ldb, kBK, BN, 2);
    else ok = encode_tmap_2d(&tmB, B, K + xb, N, ldb, 64, kBK, 2);
    if (!ok) return CAI_K_BAD_ARG;
    p.status = status_words(dev);
    p.stamps = p.mode != kGemmPlain ? g_stamp_buf[dev & 63] : nullptr;
    CUtensorMap tmA2 = tmA;
    if (p.mode == kGemmAllGatherA &&
        !encode_tmap_2d(&tmA2, p.pt.base[p.pt.rank] + p.src_off, p.rows_per_rank, K, p.ld_src, kBK, kBM, 2))
        return CAI_K_BAD_ARG;
    if (p.mode == kGemmReduceScatter) {
        if (BN == 256) return launch_gemm<256, 4, true>(tmA, tmB, tmA2, p, sms, st);
        return launch_gemm<128, 6, true>(tmA, tmB, tmA2, p, sms, st);
    }
    if (BN == 256) return launch_gemm<256, 4, false>(tmA, tmB, tmA2, p, sms, st);
    return launch_gemm<128, 6, false>(tmA, tmB, tmA2, p, sms, st);
}

static void plain_params(GemmParams& p) {
    p.mode = kGemmPlain;
    p.group_kind = 0; p.n_copy = 0; p.rows_per_rank = 0; p.m_rot = 0;
    p.epoch_base = nullptr; p.seq = 0; p.src_off = 0; p.stage_off = 0; p.a_full = nullptr; p.ld_src = 0;
    p.pt = PeerTable{};
    p.seg_counts = nullptr; p.seg_rows = 0; p.seg_mode = 0;
    p.groups = 1; p.grp_a = p.grp_b = p.grp_c = 0; p.grp_seg = 0;
    p.gat = GatherJob{}; p.b_elem_off = 0; p.ldb = 0; p.stamps = nullptr; p.tail_start = 0x7fffffff;
    p.R = nullptr; p.ldr = 0; p.alpha = 1.f; p.epi = CAI_EPI_BF16; p.a_mn = 0;
}

}  // namespace cai

using namespace cai;

CAI_API int cai_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                          long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                          int b_mn_major, int epi, float alpha, int sm_limit, void* stream) {
    return cai_gemm_bf16_seg(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn_major, b_mn_major, epi, alpha, nullptr, 0, 0,
                             sm_limit, stream);
}

CAI_API int cai_gemm_bf16_seg(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                              long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                              int b_mn_major, int epi, float alpha, const int* seg_counts, int seg_rows, int seg_mode,
                              int sm_limit, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return CAI_K_OK;
    if (seg_mode && (!seg_counts || seg_rows <= 0 || seg_rows % 128 || seg_mode > 2)) {
        set_last_error("gemm: segmented form needs counts and a slab size that is a multiple of 128");
        return CAI_K_BAD_ARG;
    }
    if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3) || epi < 0 || epi > CAI_EPI_SWIGLU_BWD) {
        set_last_error("gemm: N, lda, ldb must be multiples of 8 (N=%d lda=%lld ldb=%lld ldc=%lld epi=%d)", N,
                       lda, ldb, ldc, epi);
        return CAI_K_BAD_ARG;
    }
    if ((epi == CAI_EPI_BF16 || epi == CAI_EPI_BF16_RESIDUAL) && (ldc & 7)) {
        set_last_error("gemm: bf16 output needs ldc %% 8 == 0");
        return CAI_K_BAD_ARG;
    }
    if (epi == CAI_EPI_BF16_RESIDUAL && (!R || (ldr & 7))) {
        set_last_error("gemm: residual epilogue needs R with ldr %% 8 == 0");
        return CAI_K_BAD_ARG;
    }
    if ((epi == CAI_EPI_SWIGLU || epi == CAI_EPI_SWIGLU_BWD) && (!R || (ldr & 7) || (ldc & 7) || seg_mode == 2)) {
        set_last_error("gemm: SwiGLU epilogues need the second tensor R with ldr %% 8 == 0 and ldc %% 8 == 0");
        return CAI_K_BAD_ARG;
    }
    if (epi == CAI_EPI_SWIGLU && (b_mn_major || (N % 256))) {
        set_last_error("gemm: fused SwiGLU needs B stored [2F, K] with F a multiple of 128 (N=%d)", N);
        return CAI_K_BAD_ARG;
    }
    GemmParams p;
    plain_params(p);
    p.M = M; p.N = N; p.K = K;
    p.a_mn = a_mn_major ? 1 : 0;
    p.b_mn = b_mn_major ? 1 : 0;
    p.epi = epi;
    p.alpha = alpha;
    p.C = C; p.R = R;
    p.ldc = ldc; p.ldr = ldr;
    p.seg_counts = seg_counts; p.seg_rows = seg_rows; p.seg_mode = seg_mode;
    return gemm_dispatch(A, B, lda, ldb, p, sm_limit, reinterpret_cast<cudaStream_t>(stream));
}

CAI_API int cai_gemm_bf16_grouped(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int epi, const int* seg_counts, int seg_rows,
                                  int seg_mode, int groups, long long grp_a, long long grp_b, long long grp_c, int grp_seg,
                                  void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return CAI_K_OK;
    if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3) || (epi != CAI_EPI_BF16 && (epi != CAI_EPI_F32) && epi != CAI_EPI_F32_ACCUM) ||
        (epi == CAI_EPI_BF16 && (ldc & 7)) || (seg_mode && (!seg_counts || seg_rows <= 0 || seg_rows % 128 || seg_mode > 2)) ||
        ((a_mn_major || b_mn_major) && groups > 1 && (K % kBK))) {
        set_last_error("gemm_grouped: bad arguments (M=%d N=%d K=%d groups=%d)", M, N, K, groups);
        return CAI_K_BAD_ARG;
    }
    GemmParams p;
    plain_params(p);
    p.M = M; p.N = N; p.K = K;
    p.a_mn = a_mn_major ? 1 : 0;
    p.b_mn = b_mn_major ? 1 : 0;
    p.epi = epi;
    p.C = C; p.ldc = ldc;
    p.seg_counts = seg_counts; p.seg_rows = seg_rows; p.seg_mode = seg_mode;
    p.groups = groups; p.grp_a = grp_a; p.grp_b = grp_b; p.grp_c = grp_c; p.grp_seg = grp_seg;
    return gemm_dispatch(A, B, lda, ldb, p, 0, reinterpret_cast<cudaStream_t>(stream));
}

// y[T,N] = concat_rows(x_local of every member)[T,K] * op(B); also leaves the gathered rows in a_full.
int cai_fused_ag_gemm(const PeerTable& pt, int group_kind, unsigned long long src_off, long long ld_src, void* a_full,
                      const void* B, void* C, int T, int N, int K, long long ldb, long long ldc, int b_mn,
                      int rows_per_rank, const uint32_t* epoch_base, uint32_t seq, int n_copy, cudaStream_t st,
                      int epi, const void* R, long long ldr) {
    if (rows_per_rank % kBM || rows_per_rank * pt.size != T || (N & 7) || (K & 7) || (ldb & 7) || (ldc & 7) ||
        T / kBM > static_cast<int>(kSigLocalSlots)) {
        set_last_error("ag_gemm: rows per member must be a multiple of 128 (T=%d rows_per_rank=%d)", T, rows_per_rank);
        return CAI_K_BAD_ARG;
    }
    if ((epi != CAI_EPI_BF16 && epi != CAI_EPI_SWIGLU && epi != CAI_EPI_SWIGLU_BWD) ||
        (epi != CAI_EPI_BF16 && (!R || (ldr & 7))) || (epi == CAI_EPI_SWIGLU && (b_mn || (N % 256)))) {
        set_last_error("ag_gemm: unsupported epilogue %d for N=%d", epi, N);
        return CAI_K_BAD_ARG;
    }
    GemmParams p;
    plain_params(p);
    p.M = T; p.N = N; p.K = K;
    p.b_mn = b_mn ? 1 : 0;
    p.C = C; p.ldc = ldc;
    p.epi = epi; p.R = R; p.ldr = ldr;
    p.mode = kGemmAllGatherA;
    p.group_kind = group_kind;
    if (n_copy <= 0) {
        // Sixteen copy CTAs already move what the fabric gives when every member pulls at once (measured with the
        // per-CTA stamps on 4 GPUs: 50 MB of remote rows in ~110 us with 16 CTAs and with 25); more only take SMs from
        // the GEMM. When the GEMM has fewer tiles than SMs the idle SMs copy too (up to 32).
        const int sms = sm_count(current_device());
        const int tiles = ((T + kBM - 1) / kBM) * ((N + 255) / 256);
        n_copy = sms - tiles;
        n_copy = n_copy < 16 ? 16 : n_copy > 32 ? 32 : n_copy;
        const int units = T / kBM;
        if (n_copy > units) n_copy = units;
    }
    p.n_copy = n_copy;
    p.rows_per_rank = rows_per_rank;
    p.m_rot = pt.rank * (rows_per_rank / kBM);  // own rows first
    p.epoch_base = epoch_base; p.seq = seq;
    p.src_off = src_off; p.ld_src = ld_src;
    p.a_full = static_cast<__nv_bfloat16*>(a_full);
    p.pt = pt;
    return gemm_dispatch(a_full, B, K, ldb, p, 0, st);
}

// out_local[T/size, N] = residual + sum over members of (A_member[T,K] * op(B_member))[my rows].
int cai_fused_gemm_rs(const PeerTable& pt, int group_kind, const void* A, const void* B, unsigned long long stage_off,
                      void* out_local, const void* residual, int T, int N, int K, long long lda, long long ldb,
                      long long ldo, long long ldr, int b_mn, int rows_per_rank, const uint32_t* epoch_base, uint32_t seq,
                      cudaStream_t st) {
    if (rows_per_rank % kBM || rows_per_rank * pt.size != T || (N & 7) || (lda & 7) || (ldb & 7) || (ldo & 7) ||
        (residual && (ldr & 7))) {
        set_last_error("gemm_rs: rows per member must be a multiple of 128 (T=%d rows_per_rank=%d)", T, rows_per_rank);
        return CAI_K_BAD_ARG;
    }
    GemmParams p;
    plain_params(p);
    p.M = T; p.N = N; p.K = K;
    p.b_mn = b_mn ? 1 : 0;
    p.C = out_local; p.ldc = ldo;
    p.R = residual; p.ldr = ldr;
    p.mode = kGemmReduceScatter;
    p.group_kind = group_kind;
    p.rows_per_rank = rows_per_rank;
    p.m_rot = ((pt.rank + 1) % pt.size) * (rows_per_rank / kBM);  // push to the other members first
    p.epoch_base = epoch_base; p.seq = seq;
    p.stage_off = stage_off;
    p.pt = pt;
    return gemm_dispatch(A, B, lda, ldb, p, 0, st);
}

// C = op(A) * op(B) (+ residual) where B is a parameter inside the staged range [lo, hi) of the sharded
// flat parameter space: the leading copy CTAs stage the whole range (every later GEMM of the layer
// reads the staged copy), the compute CTAs start as soon as the slots under their B tile are there.
int cai_fused_gather_gemm(const PeerTable& pt, const cai::GatherJob& job_in, const void* A, const void* B, void* C, const void* R,
                          int M, int N, int K, long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int b_mn,
                          int epi, float alpha, const uint32_t* epoch_base, uint32_t seq, cudaStream_t st) {
    GatherJob job = job_in;
    gather_job_finish(job);
    const long long b_off = static_cast<const __nv_bfloat16*>(B) - job.dst;
    if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3) || b_off < 0 || b_off >= job.hi - job.lo || job.nslots < 1 ||
        job.nslots > static_cast<int>(kSigLocalSlots) || job.n_copy < 1) {
        set_last_error("gather_gemm: B must lie inside the staged range (offset %lld of %lld)", b_off, job.hi - job.lo);
        return CAI_K_BAD_ARG;
    }
    GemmParams p;
    plain_params(p);
    p.M = M; p.N = N; p.K = K;
    p.a_mn = a_mn ? 1 : 0; p.b_mn = b_mn ? 1 : 0;
    p.epi = epi; p.alpha = alpha;
    p.C = C; p.ldc = ldc; p.R = R; p.ldr = ldr;
    p.mode = kGemmGatherB;
    p.group_kind = job.group_kind;
    p.n_copy = job.n_copy;
    p.epoch_base = epoch_base; p.seq = seq;
    p.pt = pt;
    p.gat = job;
    p.b_elem_off = b_off;
    p.ldb = ldb;
    return gemm_dispatch(A, B, lda, ldb, p, 0, st);
}

// Per-CTA phase stamps of the fused GEMM modes: `buf` holds 8 x 256 uint64 (device memory, zeroed by the caller) or is
// null to switch the stamps off. Word layout: kernel entry, first tile ready, first accumulator, last epilogue,
// reduce start, reduce flags seen, CTA end, copy CTA done (globaltimer ns). Used by cai_b200/parallel/fused_bench.py.
CAI_API int cai_fused_debug_stamps(void* buf) {
    g_stamp_buf[current_device() & 63] = static_cast<unsigned long long*>(buf);
    return 0;
}

// ---- C forms of the fused GEMMs with explicit member bases (tests, micro-benchmarks, other runtimes).
// bases[rank] is the local arena; sig_off is the arena offset of the signal block; epoch_base a device word.
static PeerTable peer_table_of(void* const* bases, int rank, int size, unsigned long long sig_off) {
    PeerTable pt{};
    for (int i = 0; i < size && i < kMaxPeers; ++i) pt.base[i] = static_cast<uint8_t*>(bases[i]);
    pt.rank = rank;
    pt.size = size;
    pt.sig_off = sig_off;
    return pt;
}

CAI_API int cai_fused_ag_gemm_c(void* const* bases, int rank, int size, unsigned long long sig_off, int group_kind,
                                unsigned long long src_off, long long ld_src, void* a_full, const void* B, void* C, int T, int N,
                                int K, long long ldb, long long ldc, int b_mn, const uint32_t* epoch_base, uint32_t seq, int n_copy,
                                void* stream) {
    if (size < 1 || size > kMaxPeers || T % size) return CAI_K_BAD_ARG;
    return cai_fused_ag_gemm(peer_table_of(bases, rank, size, sig_off), group_kind, src_off, ld_src, a_full, B, C, T, N, K, ldb, ldc,
                             b_mn, T / size, epoch_base, seq, n_copy, static_cast<cudaStream_t>(stream), CAI_EPI_BF16, nullptr, 0);
}

CAI_API int cai_fused_gemm_rs_c(void* const* bases, int rank, int size, unsigned long long sig_off, int group_kind, const void* A,
                                const void* B, unsigned long long stage_off, void* out_local, const void* residual, int T, int N,
                                int K, long long lda, long long ldb, long long ldo, long long ldr, int b_mn,
                                const uint32_t* epoch_base, uint32_t seq, void* stream) {
    if (size < 1 || size > kMaxPeers || T % size) return CAI_K_BAD_ARG;
    return cai_fused_gemm_rs(peer_table_of(bases, rank, size, sig_off), group_kind, A, B, stage_off, out_local, residual, T, N, K, lda,
                             ldb, ldo, ldr, b_mn, T / size, epoch_base, seq, static_cast<cudaStream_t>(stream));
}
