// Tensor-core GEMM with the fused epilogue for sm_100a: tcgen05.mma with TMEM
// accumulators, operands staged in shared memory by TMA, warp-specialised and
// persistent.
//
//   C <- epi(alpha * (A @ B) + beta * C + bias)
//     f16 / bf16 inputs -> fp32 accumulate -> f32 | f16 | bf16 output   (kind::f16)
//     f32 inputs computed as TF32 -> fp32 accumulate -> f32 output      (kind::tf32)
//     s8 / u8 inputs -> int32 accumulate -> s32 output, exact           (kind::i8)
//
// It replaces what the reference generates from its tensorization and caching
// passes (accera/transforms/src/exec/ExecutionPlanToAffineLoweringPass.cpp:
// 5986-6533 and 2663-2883): per-warp wmma fragments fed by cooperative
// global->shared copies with __syncthreads.  The fused epilogue corresponds to the
// reference's fragment ops applied before store_matrix_sync
// (accera/acc-translate/src/Target/Cpp/CppPrinterUtils.h:630-655), applied here
// once per output tile after the whole K accumulation.
//
// Layout contract: each operand is K-contiguous (row-major A, column-major B: "K-major", loaded without
// transposition) or, for 16-bit and 8-bit types, M / N-contiguous (column-major A, row-major B: "MN-major"
// shared-memory descriptors), with 16-byte aligned rows.
//
// Kernel structure (one CTA per SM, 192 or 320 threads, or CTA pairs with cta_group::2):
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of a
//               128-byte-wide K slab of A (128 rows) and B (256 rows, or 128 per CTA
//               of a pair) into a ring of shared-memory stages (128B swizzle)
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (M=128|256, N=256,
//               K=32 bytes per instruction), commits to the stage's "empty"
//               mbarrier, and after the last K slab to the accumulator's "full" one
//   warps 2..5  epilogue: tcgen05.ld the 128 x 256 accumulator (each warp its own 32
//               TMEM lanes; launches with a short K loop run warps 2..9, two per lane
//               quarter, each taking half of the columns),
//               scale / add C / bias / ReLU / convert, then one of three ways out:
//               shared-memory boxes stored by TMA (the default), boxes the warps move
//               themselves with the old C copied in ahead of use (short K loops with
//               beta != 0), or 16-byte stores straight from registers (column-major C)
// A launch that writes C to several replicas (other GPUs' memory) can set its last
// CTAs aside to forward finished tiles instead of computing (copy_tiles).
// Two TMEM accumulators (2 x 256 columns) let the epilogue of tile i overlap the
// main loop of tile i+1.  Tiles are visited in groups of rows so that the CTAs
// running at the same time share A and B panels in L2.
//
// Every mbarrier wait is bounded: when a wait runs out the kernel records where
// in the status buffer, all roles leave their loops, TMEM is freed and the kernel
// returns; the host reports ACCB_ERR_TIMEOUT.  Nothing traps.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "accb_internal.h"

namespace accb {
namespace {

constexpr int kBlockM = 128;          // accumulator rows per CTA (TMEM lanes)
constexpr int kBlockN = 256;          // widest accumulator tile (UMMA N); kernels are also built for 128 columns
constexpr int kSlabBytes = 128;       // bytes of K per stage row: one 128B swizzle atom
constexpr int kMmaKBytes = 32;        // bytes of K one tcgen05.mma consumes
constexpr int kThreads = 192;          // producer warp, MMA warp, four epilogue warps
constexpr int kEpiWarps = 4;
constexpr int kThreadsWide = 320;      // with eight epilogue warps (launches whose epilogue shows: see UmmaParams::epi_warps)
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address (rank 0 of a pair)

enum { KIND_F16 = 0, KIND_TF32 = 1, KIND_I8 = 2 };

// where a bounded wait gave up (status word 1, bits 31..24)
enum { SITE_PRODUCER_EMPTY = 1, SITE_MMA_FULL = 2, SITE_MMA_TMEM_EMPTY = 3, SITE_EPI_TMEM_FULL = 4, SITE_COPY_TILE = 5 };

// BN = accumulator columns per tile: 256, or 128 for problems whose tile count fills the SMs badly at 256
template <bool TWO_SM, int BN> struct SmemPlan {
    static constexpr int kABytes = kBlockM * kSlabBytes;                  // 16 KB
    static constexpr int kBBytes = (TWO_SM ? BN / 2 : BN) * kSlabBytes;   // 8 to 32 KB
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 256;
    // epilogue staging for TMA stores: per epilogue warp two boxes of 32 rows x 128 bytes (128-byte swizzle)
    static constexpr int kStoreBoxBytes = 32 * 128;
    static constexpr int kStoreBytes = kEpiWarps * 2 * kStoreBoxBytes;
    // as many stages as fit beside the staging boxes: 4 (1 SM, 256), 6 (pair, 256 / 1 SM, 128), 8 (pair, 128)
    static constexpr int kBudget = 227 * 1024 - 1024 - kBarrierBytes - kStoreBytes;   // 227 KB per CTA on sm_100
    static constexpr int kStages = kBudget / kStageBytes > 8 ? 8 : kBudget / kStageBytes;
    // launches that also bring the old C in through the staging boxes (c_in) use four boxes per epilogue warp; the
    // second kStoreBytes are taken from the end of the operand ring: 5, 6, 3 and 5 stages remain
    static constexpr int kCinBoxes = 4;
    static constexpr int kCinStages = kStages - (kStoreBytes + kStageBytes - 1) / kStageBytes;
    static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + kStoreBytes + 1024;   // +1024: manual alignment
    static constexpr int kTmemCols = 2 * BN;   // two accumulators of BN fp32 columns (a power of two >= 32)
};

constexpr int kMaxReplicas = 8;
constexpr int kPeerStoreDefault = 0;   // how replicas in peer memory are written unless overridden: 0 TMA stores, 1 register stores
struct CReplicaMaps { CUtensorMap m[kMaxReplicas]; };   // tensor maps of the C replicas (TMA-store epilogue)

struct UmmaParams {
    int64_t m, n, k;
    int64_t cs0, cs1;       // C strides in elements
    float alpha, beta;
    int relu;
    uint32_t idesc;         // tcgen05 instruction descriptor
    int elem_bytes;         // bytes per A/B element
    int tiles_m, tiles_n;   // tiles_m counts units of 128 rows (1 CTA) or 256 rows (pair)
    int group_m;            // tile rows visited together (L2 reuse)
    int hint_a, hint_b;     // L2 eviction priority of the operand loads: 0 normal, 1 evict-first, 2 evict-last
    int c_stream;           // read / write C with streaming (evict-first) accesses
    int tma_store;          // epilogue goes through shared memory and TMA stores (row-major C with 16-byte pitch)
    int n_replicas;         // number of C replicas the result is stored to (1 = just C); replicas may be peer memory
    int a_mn, b_mn;         // operand is MN-contiguous in global memory (column-major A / row-major B)
    int pace_pct;           // 0 = off; else a CTA starts loading its i-th tile only once pace_pct % of all CTAs'
                            // (i-1)-th tiles have been loaded (or a few microseconds have passed)
    int* pace;              // this launch's progress counter
    int* status;
    // batched GEMM: `batch` problems of the same shape in one launch; tile index = problem * tiles_m * tiles_n + tile.
    // A batched operand has a rank-3 tensor map whose outermost coordinate is the problem; an operand shared
    // by all problems keeps its rank-2 map.  C of problem b starts c_bs elements after that of problem b - 1.
    int batch;
    int a_batched, b_batched;
    int64_t c_bs;
    int verbose;            // host only: print the launch plan to stderr
    int pdl;                // host only: launch with programmatic stream serialization
    int launch_id;          // non-zero id of this launch: failures recorded in the status buffer carry it
    unsigned long long wait_ns;   // limit of every bounded wait, in nanoseconds of the global timer
    int drop_commit;        // self-test of the time-out path: the commit completing each CTA's last accumulator is left out
    int peer_store;         // replicas 1.. are written with 16-byte register stores read back from the staging box
                            // (replica 0 keeps its TMA store); 0 = one TMA store per replica
    void* peer_c[kMaxReplicas - 1];   // base pointers of replicas 1.. (peer_store and copy CTAs)
    int copy_ctas;          // > 0: the last copy_ctas CTAs of the grid compute nothing; they forward every finished tile
                            // of the local C to the replicas (see copy_tiles).  The computing CTAs then store to C only.
    int* tile_flags;        // copy_ctas > 0: one counter per tile, bumped by every epilogue warp once its part of the
                            // tile is in C; zeroed by the host before the launch
    int lsu_stage;          // staged epilogue whose boxes are moved between shared and global memory by the warp itself
                            // (coalesced 16-byte accesses) instead of by TMA; taken for short K loops, where a TMA store or
                            // load of C queues behind the operand loads of several pipeline stages
    int c_in;               // lsu_stage with beta != 0: the old C is copied into the staging boxes boxes ahead (cp.async,
                            // also across tiles) instead of being read row by row when it is needed
    int epi_warps;          // 4, or 8 with lsu_stage: two warps per TMEM lane quarter, each taking half of the tile's columns.
                            // An epilogue warp is alone on its scheduler and bound by instruction latency (measured 0.6 us
                            // per 32-column chunk); where a CTA's last epilogue is a large part of the launch, a second
                            // warp per scheduler halves it
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// arrive on a barrier addressed in the cluster window (own CTA or the pair's rank 0)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false when it gave up: after `wait_ns` (a second unless the caller asked otherwise), or as
// soon as a CTA of THIS launch has recorded a failure.  The first failure of a launch is recorded with the launch's
// id; a record left by an earlier launch is not this launch's business and neither stops it nor is overwritten.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int* status, int launch_id, unsigned long long wait_ns,
                                            int site, int detail)
{
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 0x3f) == 0x3f) {
            if (*(volatile int*)(status + ST_GEMM_ID) == launch_id) return false;   // another CTA of this launch already failed
            if (global_timer_ns() - t0 > wait_ns) {
                atomicAdd(status + ST_GEMM_COUNT, 1);
                if (atomicCAS(status + ST_GEMM_ID, 0, launch_id) == 0) {
                    status[ST_GEMM_SITE] = (site << 24) | (int)(blockIdx.x & 0xffffff);
                    status[ST_GEMM_STEP] = detail;
                }
                return false;
            }
        }
    }
}
struct WaitCtx { int* status; int launch_id; unsigned long long wait_ns; };
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, int site, int detail)
{
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, w.status, w.launch_id, w.wait_ns, site, detail);
}

// L2 eviction-priority policy for the operand loads; 0 = none (the plain load form is used)
__device__ __forceinline__ uint64_t make_l2_policy(int hint)
{
    uint64_t pol = 0;
    if (hint == 1) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    else if (hint == 2) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, uint64_t pol)
{
    if (pol == 0)
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "l"(pol)
            : "memory");
}
// CTA-pair form: the transaction bytes are signalled on the barrier of the pair's rank-0 CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, uint64_t pol)
{
    if (pol == 0)
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar & kPeerMask), "r"(c0), "r"(c1)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar & kPeerMask), "r"(c0), "r"(c1), "l"(pol)
            : "memory");
}

// Rank-3 forms for batched operands: the box is [1][rows][128 bytes], laid out in shared memory like the rank-2 box
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar & kPeerMask), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// TMA store of one shared-memory box into a C replica (rows / columns outside the tensor are clipped)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes
// with the 128-byte swizzle (what TMA writes): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // layout: 128-byte swizzle
    return d;
}

// MN-major operand tile as TMA writes it from an MN-contiguous array: boxes of [k rows][128 bytes of MN] with
// the 128-byte swizzle; 8 k-rows form one 1024-byte swizzle atom (stride byte offset), consecutive 128-byte
// MN blocks are `mn_block_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t mn_block_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)((mn_block_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int KIND, bool TWO_SM>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (!TWO_SM) {
        if constexpr (KIND == KIND_F16)
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
        else if constexpr (KIND == KIND_TF32)
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
        else
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        if constexpr (KIND == KIND_F16)
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
        else if constexpr (KIND == KIND_TF32)
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
        else
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                         ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    }
}

// Make `bar` (same offset in every CTA of cta_mask) complete once all tcgen05.mma
// issued so far by this thread have finished reading shared memory / writing TMEM.
template <bool TWO_SM>
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    if constexpr (!TWO_SM) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    } else {
        const uint16_t mask = 3;
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(bar), "h"(mask) : "memory");
    }
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Waits for this thread's outstanding tcgen05.ld.  The registers of the load are passed through the statement so
// that the compiler orders every use of them after the wait (a load may be issued well before its data is needed).
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :
        : "memory");
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// tile index -> (tile row, tile column): groups of `group_m` tile rows, rows fastest inside a group.
// (Cutting the columns into bands as well, so that a band of B could stay in L2 while row groups stream past it,
// was measured and changes neither the DRAM traffic - 2.76 to 3.16 GB per launch at 16384 x 8192 x 8192 for
// every band shape tried, against 2.89 GB without bands - nor the run time: the 74 tiles in flight at any moment
// already span more of A and B than stays resident in L2 between two rounds.)
__device__ __forceinline__ void tile_coords(int t, const UmmaParams& p, int& tm, int& tn)
{
    const int group_size = p.group_m * p.tiles_n;
    const int group = t / group_size;
    const int first_m = group * p.group_m;
    const int rows = min(p.tiles_m - first_m, p.group_m);
    const int in = t - group * group_size;
    tm = first_m + in % rows;
    tn = in / rows;
}

// batched launches: tile index -> (problem, tile row, tile column)
__device__ __forceinline__ void tile_coords_batched(int t, const UmmaParams& p, int& problem, int& tm, int& tn)
{
    problem = 0;
    if (p.batch > 1) {
        const int per = p.tiles_m * p.tiles_n;
        problem = t / per;
        t -= problem * per;
    }
    tile_coords(t, p, tm, tn);
}

// 16-byte C accesses, optionally streaming (evict-first) so that C does not displace A / B panels in L2
template <typename V> __device__ __forceinline__ V ld_c(const V* p, bool stream) { return stream ? __ldcs(p) : *p; }
template <typename V> __device__ __forceinline__ void st_c(V* p, const V& v, bool stream) { if (stream) __stcs(p, v); else *p = v; }

template <typename TC, typename ACC>
__device__ __forceinline__ void epilogue_row(const uint32_t (&acc)[32], TC* __restrict__ crow, int64_t col0, int ncols,
                                             bool vec_ok, int64_t cs1, const float* __restrict__ bias,
                                             const UmmaParams& p)
{
    // crow points at C[row, 0]; this thread owns columns [col0, col0 + 32) of which ncols are inside the matrix
    if constexpr (std::is_same<ACC, int>::value) {
        int v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (int)acc[j];
        if (vec_ok && ncols == 32) {
            int4* dst = reinterpret_cast<int4*>(crow + col0);
            if (p.beta != 0.0f) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    int4 o = ld_c(dst + q, p.c_stream);
                    v[4 * q] += o.x; v[4 * q + 1] += o.y; v[4 * q + 2] += o.z; v[4 * q + 3] += o.w;
                }
            }
            if (p.relu) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = max(v[j], 0);
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) st_c(dst + q, make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]), p.c_stream);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < ncols) {
                    TC* d = crow + (col0 + j) * cs1;
                    int x = v[j];
                    if (p.beta != 0.0f) x += (int)*d;
                    if (p.relu) x = max(x, 0);
                    *d = (TC)x;
                }
            }
        }
    } else {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
        if (p.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
        }
        if (vec_ok && ncols == 32) {
            if constexpr (std::is_same<TC, float>::value) {
                float4* dst = reinterpret_cast<float4*>(crow + col0);
                if (p.beta != 0.0f) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 o = ld_c(dst + q, p.c_stream);
                        v[4 * q] += p.beta * o.x; v[4 * q + 1] += p.beta * o.y;
                        v[4 * q + 2] += p.beta * o.z; v[4 * q + 3] += p.beta * o.w;
                    }
                }
                if (bias) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += __ldg(bias + col0 + j);
                }
                if (p.relu) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) st_c(dst + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]), p.c_stream);
            } else {
                // 16-bit outputs: 8 elements per 16-byte vector
                uint4* dst = reinterpret_cast<uint4*>(crow + col0);
                if (p.beta != 0.0f) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o = ld_c(dst + q, p.c_stream);
                        const TC* h = reinterpret_cast<const TC*>(&o);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[8 * q + e] += p.beta * (float)h[e];
                    }
                }
                if (bias) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += __ldg(bias + col0 + j);
                }
                if (p.relu) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    TC* h = reinterpret_cast<TC*>(&o);
#pragma unroll
                    for (int e = 0; e < 8; ++e) h[e] = (TC)v[8 * q + e];
                    st_c(dst + q, o, p.c_stream);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < ncols) {
                    TC* d = crow + (col0 + j) * cs1;
                    float x = v[j];
                    if (p.beta != 0.0f) x += p.beta * (float)*d;
                    if (bias) x += __ldg(bias + col0 + j);
                    if (p.relu) x = fmaxf(x, 0.0f);
                    *d = (TC)x;
                }
            }
        }
    }
}

// Same arithmetic as epilogue_row, but the 32 results of this thread's row go to `srow` in shared memory
// (the staging box of a TMA store).  C is only read (beta != 0) where it exists; values computed for
// rows / columns outside the matrix are never stored, the TMA store clips them.
template <typename TC, typename ACC>
__device__ __forceinline__ void epilogue_to_smem(const uint32_t (&acc)[32], const TC* __restrict__ crow, bool row_ok,
                                                 int64_t col0, int ncols, bool c_vec, const float* __restrict__ bias,
                                                 const UmmaParams& p, uint8_t* srow, int slot0, int lane7)
{
    // srow: this thread's 128-byte row of the staging box; the 32 results occupy 16-byte slots
    // slot0 .. slot0 + (32 * sizeof(TC) / 16) - 1, each stored at slot ^ (row % 8): the 128-byte swizzle of
    // the TMA store map, which also makes the 8 rows of a store phase hit 8 different bank groups
    const bool full = (ncols == 32);
    if constexpr (std::is_same<ACC, int>::value) {
        int v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (int)acc[j];
        if (p.beta != 0.0f && row_ok) {
            if (c_vec && full) {
                const int4* src = reinterpret_cast<const int4*>(crow + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int4 o = ld_c(src + q, p.c_stream);
                    v[4 * q] += o.x; v[4 * q + 1] += o.y; v[4 * q + 2] += o.z; v[4 * q + 3] += o.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += (int)crow[col0 + j];
            }
        }
        if (p.relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = max(v[j], 0);
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<int4*>(srow + (((slot0 + q) ^ lane7) << 4)) = make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
        if (p.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
        }
        if (p.beta != 0.0f && row_ok) {
            if (c_vec && full) {
                if constexpr (sizeof(TC) == 4) {
                    const float4* src = reinterpret_cast<const float4*>(crow + col0);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float4 o = ld_c(src + q, p.c_stream);
                        v[4 * q] += p.beta * o.x; v[4 * q + 1] += p.beta * o.y;
                        v[4 * q + 2] += p.beta * o.z; v[4 * q + 3] += p.beta * o.w;
                    }
                } else {
                    const uint4* src = reinterpret_cast<const uint4*>(crow + col0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 o = ld_c(src + q, p.c_stream);
                        const TC* h = reinterpret_cast<const TC*>(&o);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[8 * q + e] += p.beta * (float)h[e];
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += p.beta * (float)crow[col0 + j];
            }
        }
        if (bias) {
            if (full) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __ldg(bias + col0 + j);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __ldg(bias + col0 + j);
            }
        }
        if (p.relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
        }
        if constexpr (sizeof(TC) == 4) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(srow + (((slot0 + q) ^ lane7) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 o;
                TC* h = reinterpret_cast<TC*>(&o);
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = (TC)v[8 * q + e];
                *reinterpret_cast<uint4*>(srow + (((slot0 + q) ^ lane7) << 4)) = o;
            }
        }
    }
}

// The staged epilogue when the old C is already in the staging box (brought there by a TMA load): this thread's
// 32 results are combined with the C values found in their own 16-byte slots and written back over them.  Rows and
// columns outside the matrix were zero-filled by the load and are clipped by the store.
template <typename TC, typename ACC>
__device__ __forceinline__ void epilogue_inplace(const uint32_t (&acc)[32], int64_t col0, int ncols,
                                                 const float* __restrict__ bias, const UmmaParams& p, uint8_t* srow,
                                                 int slot0, int lane7)
{
    if constexpr (std::is_same<ACC, int>::value) {
        int v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (int)acc[j];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int4 o = *reinterpret_cast<const int4*>(srow + (((slot0 + q) ^ lane7) << 4));
            v[4 * q] += o.x; v[4 * q + 1] += o.y; v[4 * q + 2] += o.z; v[4 * q + 3] += o.w;
        }
        if (p.relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = max(v[j], 0);
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<int4*>(srow + (((slot0 + q) ^ lane7) << 4)) = make_int4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
        if (p.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
        }
        if constexpr (sizeof(TC) == 4) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 o = *reinterpret_cast<const float4*>(srow + (((slot0 + q) ^ lane7) << 4));
                v[4 * q] += p.beta * o.x; v[4 * q + 1] += p.beta * o.y;
                v[4 * q + 2] += p.beta * o.z; v[4 * q + 3] += p.beta * o.w;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 o = *reinterpret_cast<const uint4*>(srow + (((slot0 + q) ^ lane7) << 4));
                const TC* h = reinterpret_cast<const TC*>(&o);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[8 * q + e] += p.beta * (float)h[e];
            }
        }
        if (bias) {
            if (ncols == 32) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __ldg(bias + col0 + j);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __ldg(bias + col0 + j);
            }
        }
        if (p.relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
        }
        if constexpr (sizeof(TC) == 4) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(srow + (((slot0 + q) ^ lane7) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 o;
                TC* h = reinterpret_cast<TC*>(&o);
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = (TC)v[8 * q + e];
                *reinterpret_cast<uint4*>(srow + (((slot0 + q) ^ lane7) << 4)) = o;
            }
        }
    }
}

template <int KIND> struct ElemBytes { static constexpr int value = (KIND == KIND_F16) ? 2 : (KIND == KIND_TF32) ? 4 : 1; };

// One TMA box of an operand.  BATCHED launches address a batched operand through its rank-3 map (the problem is
// the outermost coordinate, no L2 hint); an operand shared by all problems keeps the rank-2 form.
template <bool TWO_SM, bool BATCHED>
__device__ __forceinline__ void load_box(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                         int problem, int batched_operand, uint64_t pol)
{
    if (BATCHED && batched_operand) {
        if constexpr (TWO_SM) tma_load_3d_pair(dst, map, bar, c0, c1, problem);
        else tma_load_3d(dst, map, bar, c0, c1, problem);
    } else {
        if constexpr (TWO_SM) tma_load_2d_pair(dst, map, bar, c0, c1, pol);
        else tma_load_2d(dst, map, bar, c0, c1, pol);
    }
}

// Loads k-block `kb` of this CTA's A rows and B rows into one pipeline stage.  The operand layouts are template
// parameters so that every box count, offset and coordinate step below is a compile-time constant.
//   K-major operand:  one box [rows][128 B of K]
//   MN-major operand: one box [k rows][128 B of M / N] per 128-byte block of the tile's M / N extent, stacked
template <int KIND, bool TWO_SM, int BN, bool A_MN, bool B_MN, bool BATCHED>
__device__ __forceinline__ void load_stage(const CUtensorMap* map_a, const CUtensorMap* map_b, uint32_t sa, uint32_t sb,
                                           uint32_t bar, int kb, int row_a, int row_b, int problem, int a_batched,
                                           int b_batched, uint64_t pol_a, uint64_t pol_b)
{
    constexpr int SE = kSlabBytes / ElemBytes<KIND>::value;      // elements in 128 bytes
    constexpr int kRowsB = TWO_SM ? BN / 2 : BN;
    constexpr uint32_t kBoxBytes = (uint32_t)(kSlabBytes * SE);  // one MN-major box
    if constexpr (!A_MN) {
        load_box<TWO_SM, BATCHED>(sa, map_a, bar, kb * SE, row_a, problem, a_batched, pol_a);
    } else {
#pragma unroll
        for (int blk = 0; blk < kBlockM / SE; ++blk)
            load_box<TWO_SM, BATCHED>(sa + blk * kBoxBytes, map_a, bar, row_a + blk * SE, kb * SE, problem, a_batched, pol_a);
    }
    if constexpr (!B_MN) {
        load_box<TWO_SM, BATCHED>(sb, map_b, bar, kb * SE, row_b, problem, b_batched, pol_b);
    } else {
        static_assert(kRowsB % SE == 0 || !B_MN, "an MN-major B box is 128 bytes of N wide");
#pragma unroll
        for (int blk = 0; blk < kRowsB / SE; ++blk)
            load_box<TWO_SM, BATCHED>(sb + blk * kBoxBytes, map_b, bar, row_b + blk * SE, kb * SE, problem, b_batched, pol_b);
    }
}

// Issues the tcgen05.mma instructions that consume one stage (128 bytes of K per row).
//   K-major operand:  advancing K inside the swizzle atom is +32 bytes on the descriptor's start address
//   MN-major operand: one MMA consumes (32 / element bytes) k-rows of 128 bytes each
template <int KIND, bool TWO_SM, bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_stage(uint32_t tmem_d, uint32_t sa, uint32_t sb, uint32_t idesc, bool first_kb)
{
    constexpr int EB = ElemBytes<KIND>::value;
    constexpr uint32_t kBoxBytes = (uint32_t)(kSlabBytes * (kSlabBytes / EB));
    constexpr uint64_t kStepMn = (uint64_t)(((kMmaKBytes / EB) * kSlabBytes) >> 4);
    constexpr uint64_t kStepK = (uint64_t)(kMmaKBytes >> 4);
    const uint64_t adesc = A_MN ? make_smem_desc_mn(sa, kBoxBytes) : make_smem_desc(sa);
    const uint64_t bdesc = B_MN ? make_smem_desc_mn(sb, kBoxBytes) : make_smem_desc(sb);
#pragma unroll
    for (int j = 0; j < kSlabBytes / kMmaKBytes; ++j)
        umma<KIND, TWO_SM>(tmem_d, adesc + (uint64_t)j * (A_MN ? kStepMn : kStepK), bdesc + (uint64_t)j * (B_MN ? kStepMn : kStepK),
                           idesc, (!first_kb || j > 0) ? 1u : 0u);
}

// The forwarding role of a replicated GEMM: CTAs that own no tensor-core work.  Copy CTA `copy_rank` of `n_copy`
// takes tiles copy_rank, copy_rank + n_copy, ... (the order in which the computing CTAs finish them) and moves
// each one, in bands of 32 rows, from the local C to every replica:
//   thread 0        waits until all epilogue warps of the tile have landed their part in C (a counter per tile,
//                   release / acquire), then TMA-loads the tile's bands from C (L2) into a ring of shared-memory
//                   slots, running up to a whole ring ahead of the stores
//   warps 1 .. 5    take the slots in order, read each band out of shared memory 16 bytes per thread and write
//                   it to every replica with plain stores (all of a thread's loads first, then the stores)
// Stores issued by the load/store units keep far more bytes in flight per SM than TMA stores do (measured per
// forwarding CTA with one peer: 16 GB/s with TMA stores, limited by the round trip over NVLink).
//
// Why separate CTAs: a store to another GPU waits for NVLink, and while it waits it holds up everything queued
// behind it on its SM's way out - including the operand fetches of that SM's MMA pipeline.  Measured on two
// B200s with the 8-GPU traffic pattern (7 x 128 MiB out and in per GPU, 8192^3 bf16 per step, sustained):
// stores issued by the computing CTAs' epilogues 1.55 ms per step, the same bytes stored from 16 SMs of their
// own next to a GEMM on 132 SMs 1.40 ms (the link alone needs 1.39); stores issued from the computing SMs by
// co-resident CTAs 2.03 ms.
template <typename TC, bool TWO_SM, int BN>
__device__ void copy_tiles(const UmmaParams& p, const CReplicaMaps& cmaps, uint32_t smem_base, uint8_t* smem_gen,
                           int copy_rank, int n_copy)
{
    constexpr int kRows = TWO_SM ? 2 * kBlockM : kBlockM;
    constexpr int kBoxCols = 128 / (int)sizeof(TC);              // elements per 128-byte box row
    constexpr int kBoxes = BN / kBoxCols;                        // boxes per band (32 rows x BN columns)
    constexpr uint32_t kBoxBytes = 32 * 128;
    constexpr uint32_t kSlotBytes = kBoxes * kBoxBytes;          // 16 KB (2-byte C, 256 columns) .. 32 KB
    constexpr int kSlots = (192 * 1024) / (int)kSlotBytes;       // 12 .. 6
    constexpr int kStoreWarps = kThreads / 32 - 1;
    constexpr int kStoreThreads = kStoreWarps * 32;
    constexpr int kVecPerBand = 32 * kBoxes * 8;                 // 16-byte vectors in a band
    constexpr int kVecPerThread = (kVecPerBand + kStoreThreads - 1) / kStoreThreads;
    constexpr int kPerVec = 16 / (int)sizeof(TC);
    struct BandMeta { int col, row, boxes, pad; };               // boxes < 0: no more bands
    const uint32_t bars = smem_base + (uint32_t)kSlots * kSlotBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kSlots + s); };
    volatile BandMeta* meta = reinterpret_cast<volatile BandMeta*>(smem_gen + (size_t)kSlots * kSlotBytes + 16 * kSlots);
    const WaitCtx wctx{p.status, p.launch_id, p.wait_ns};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kSlots; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), kStoreWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        if (lane != 0) return;
        // ---------------- loader ----------------
        const int num_tiles = p.tiles_m * p.tiles_n;
        const int expected = kEpiWarps * (TWO_SM ? 2 : 1);
        long long issued = 0;
        bool ok = true;
        for (int t = copy_rank; t < num_tiles && ok; t += n_copy) {
            // bounded wait for the tile (it may legitimately take most of the launch to appear)
            const unsigned long long t0 = global_timer_ns();
            for (uint32_t spin = 0;; ++spin) {
                int have;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(have) : "l"(p.tile_flags + t) : "memory");
                if (have >= expected) break;
                __nanosleep(100);
                if ((spin & 0x3f) == 0x3f) {
                    if (*(volatile int*)(p.status + ST_GEMM_ID) == p.launch_id) { ok = false; break; }
                    if (global_timer_ns() - t0 > p.wait_ns) {
                        atomicAdd(p.status + ST_GEMM_COUNT, 1);
                        if (atomicCAS(p.status + ST_GEMM_ID, 0, p.launch_id) == 0) {
                            p.status[ST_GEMM_SITE] = (SITE_COPY_TILE << 24) | (int)(blockIdx.x & 0xffffff);
                            p.status[ST_GEMM_STEP] = t;
                        }
                        ok = false;
                        break;
                    }
                }
            }
            if (!ok) break;
            // the tile was written through the async proxy and is read through it: order those reads after the acquire
            asm volatile("fence.proxy.async.global;" ::: "memory");
            int tm, tn;
            tile_coords(t, p, tm, tn);
            const int64_t row0 = (int64_t)tm * kRows;
            const int col0 = tn * BN;
            const int bands = (int)((min((int64_t)kRows, p.m - row0) + 31) / 32);
            const int nb = (int)min((int64_t)kBoxes, (p.n - col0 + kBoxCols - 1) / kBoxCols);   // boxes that touch the matrix
            for (int band = 0; band < bands; ++band, ++issued) {
                const int slot = (int)(issued % kSlots);
                if (issued >= kSlots && !mbar_wait(empty_bar(slot), (uint32_t)(((issued / kSlots) - 1) & 1), wctx, SITE_COPY_TILE, t)) { ok = false; break; }
                meta[slot].col = col0;
                meta[slot].row = (int)(row0 + band * 32);
                meta[slot].boxes = nb;
                const uint32_t dst = smem_base + (uint32_t)slot * kSlotBytes;
                mbar_arrive_expect_tx(full_bar(slot), (uint32_t)nb * kBoxBytes);   // a box clipped by the matrix edge still arrives whole
#pragma unroll
                for (int b = 0; b < kBoxes; ++b)
                    if (b < nb) tma_load_2d(dst + b * kBoxBytes, &cmaps.m[0], full_bar(slot), col0 + b * kBoxCols, (int)(row0 + band * 32), 0);
            }
        }
        // end marker for the storing warps (also after a failure, so that they leave)
        {
            const int slot = (int)(issued % kSlots);
            bool free_slot = true;
            if (issued >= kSlots && ok) free_slot = mbar_wait(empty_bar(slot), (uint32_t)(((issued / kSlots) - 1) & 1), wctx, SITE_COPY_TILE, -1);
            if (free_slot || !ok) {
                meta[slot].boxes = -1;
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_bar(slot)) : "memory");
            }
        }
        // loads still in flight after a failure: give them time to land before shared memory is released
        if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    } else {
        // ---------------- storing warps ----------------
        const int tid = (int)threadIdx.x - 32;
        const int64_t pitch = p.cs0 * (int64_t)sizeof(TC);
        for (long long j = 0;; ++j) {
            const int slot = (int)(j % kSlots);
            if (!__all_sync(0xffffffffu, mbar_wait(full_bar(slot), (uint32_t)((j / kSlots) & 1), wctx, SITE_COPY_TILE, -2))) break;
            const int nb = meta[slot].boxes;
            if (nb < 0) break;
            const int col = meta[slot].col, row = meta[slot].row;
            const uint8_t* src = smem_gen + (size_t)slot * kSlotBytes;
            uint4 v[kVecPerThread];
            int64_t off[kVecPerThread];
            const int total = 32 * nb * 8;
#pragma unroll
            for (int i = 0; i < kVecPerThread; ++i) {
                // vector -> (box, row in band, 16-byte unit): 8 consecutive threads cover one 128-byte box row
                const int vi = tid + i * kStoreThreads;
                const int b = vi >> 8, r = (vi >> 3) & 31, u = vi & 7;
                const int64_t c = (int64_t)col + b * kBoxCols + u * kPerVec;
                const bool live = vi < total && row + r < p.m && c + kPerVec <= p.n;
                off[i] = live ? (int64_t)(row + r) * pitch + c * (int64_t)sizeof(TC) : -1;
                if (live) v[i] = *reinterpret_cast<const uint4*>(src + b * kBoxBytes + r * 128 + ((u ^ (r & 7)) << 4));
            }
            for (int rep = 0; rep < p.n_replicas - 1; ++rep) {
                char* dst = reinterpret_cast<char*>(p.peer_c[rep]);
#pragma unroll
                for (int i = 0; i < kVecPerThread; ++i)
                    if (off[i] >= 0) *reinterpret_cast<uint4*>(dst + off[i]) = v[i];
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(slot)) : "memory");
        }
    }
}

template <int KIND, typename TC, bool TWO_SM, int BN>
__global__ void __launch_bounds__(kThreadsWide, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CReplicaMaps cmaps, TC* __restrict__ C, const float* __restrict__ bias,
                 const UmmaParams p)
{
    using Plan = SmemPlan<TWO_SM, BN>;
    using ACC = typename std::conditional<KIND == KIND_I8, int, float>::type;
    constexpr int kTmemCols = Plan::kTmemCols;
    constexpr int SMAX = Plan::kStages;
    // c_in (the old C copied into the staging boxes ahead of use): a tile of up to two boxes per epilogue warp (128 columns
    // of 2-byte results) fits the two boxes every launch has; wider tiles get a ring of four, for which the end of the
    // operand ring is given up
    // boxes of one tile that one epilogue warp produces, and the staging boxes it gets: all epilogue warps together have
    // kStoreBytes (every launch) or twice that (c_in with tiles wider than that, at the price of operand stages)
    const int halves = p.epi_warps / kEpiWarps;                              // 1, or 2: each warp takes half of the columns
    const int boxes_per_warp_tile = BN * (int)sizeof(TC) / 128 / halves;
    const int base_boxes = 2 / halves;                                       // boxes per warp inside kStoreBytes
    const int cin_boxes = (boxes_per_warp_tile <= base_boxes) ? base_boxes : 2 * base_boxes;
    const int S = (p.c_in && cin_boxes > base_boxes) ? Plan::kCinStages : SMAX;
    constexpr int kCtas = TWO_SM ? 2 : 1;

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128B swizzle pattern shared by TMA and the MMA descriptors
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + SMAX * Plan::kStageBytes + Plan::kStoreBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (SMAX + s); };
    auto tmem_full_bar = [&](int b) { return bars + 8u * (2 * SMAX + b); };
    auto tmem_empty_bar = [&](int b) { return bars + 8u * (2 * SMAX + 2 + b); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_gen + SMAX * Plan::kStageBytes + Plan::kStoreBytes + 8 * (2 * SMAX + 4));
    // gave_up[r] != 0: a bounded wait of the CTA with rank r in the pair ran out.  Each CTA keeps a copy of both
    // words (a CTA that gives up also writes its word into its partner's copy), so that after the closing barrier
    // both CTAs of a pair take the same teardown path without touching global memory.
    volatile uint32_t* gave_up = tmem_holder + 2;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const WaitCtx wctx{p.status, p.launch_id, p.wait_ns};
    const uint32_t rank = TWO_SM ? cluster_ctarank() : 0u;
    const bool leader = (rank == 0);

    // Programmatic dependent launch: the next kernel of the stream may be scheduled onto free SMs now and run its
    // own set-up (barriers, TMEM, descriptor prefetch) while this one computes; like this kernel below, it does not
    // touch global memory before its griddepcontrol.wait, which returns once this whole grid has finished.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // replicated GEMM with forwarding CTAs: the last copy_ctas CTAs (whole clusters) only move finished tiles
    const int compute_ctas = (int)gridDim.x - p.copy_ctas;
    if ((int)blockIdx.x >= compute_ctas) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        copy_tiles<TC, TWO_SM, BN>(p, cmaps, smem_base, smem_gen, (int)blockIdx.x - compute_ctas, p.copy_ctas);
        return;
    }

    auto record_give_up = [&]() {
        gave_up[rank] = 1u;
        if constexpr (TWO_SM) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32((const void*)(gave_up + rank))), "r"(rank ^ 1u));
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1u) : "memory");
        }
    };

    if (threadIdx.x == 0) {
        gave_up[0] = 0u;
        gave_up[1] = 0u;
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
        for (int s = 0; s < SMAX; ++s) {
            mbar_init(full_bar(s), 1);    // the producer's arrive.expect_tx (pair: rank 0's, covering both CTAs' bytes)
            mbar_init(empty_bar(s), 1);   // one tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);                    // one tcgen05.commit
            mbar_init(tmem_empty_bar(b), (uint32_t)(p.epi_warps * kCtas));   // one arrive per epilogue warp (of both CTAs)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (TWO_SM)
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32((const void*)tmem_holder)), "r"(kTmemCols) : "memory");
        else
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32((const void*)tmem_holder)), "r"(kTmemCols) : "memory");
        if constexpr (TWO_SM) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (TWO_SM) cluster_sync_all(); else __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_holder;
    // everything above touched only this CTA's shared memory and TMEM; from here on global memory is read and
    // written, which must wait for the kernel before this one in the stream (a no-op for an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int num_tiles = p.tiles_m * p.tiles_n * p.batch;
    const int num_units = compute_ctas / kCtas;
    const int unit = (int)blockIdx.x / kCtas;
    constexpr int slab_elems = kSlabBytes / ElemBytes<KIND>::value;
    const int num_kb = (int)((p.k + slab_elems - 1) / slab_elems);
    // operand layouts (bit 0: A is MN-major, bit 1: B is MN-major) and batching select one of the
    // compile-time specialised stage routines; the choice is uniform over the launch
    const int layout = (p.a_mn ? 1 : 0) | (p.b_mn ? 2 : 0);
    // an MN-major B box is 128 bytes of N: a CTA's share of B must be at least that wide (not so for 8-bit
    // operands in a 128-column pair tile; the host never selects that combination)
    constexpr bool kBMnOk = ((TWO_SM ? BN / 2 : BN) % slab_elems) == 0;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // The whole tile loop is instantiated once per operand layout / batching combination and the choice is
            // made here, once: the k loop below then contains no layout-dependent branch or arithmetic.  (The loop
            // issues two to six TMA loads per 0.3 us; anything that delays it starves the tensor pipe.)
            auto produce = [&](auto a_mn_tag, auto b_mn_tag, auto batched_tag) {
                constexpr bool A_MN = decltype(a_mn_tag)::value, B_MN = decltype(b_mn_tag)::value;
                constexpr bool BATCHED = decltype(batched_tag)::value;
                int s = 0;            // pipeline stage and its phase bit, advanced without divisions
                uint32_t ph = 0;
                bool ok = true;
                const uint64_t pol_a = make_l2_policy(p.hint_a), pol_b = make_l2_policy(p.hint_b);
                int tile_i = 0;
                bool pacing = (p.pace_pct > 0) && leader;
                for (int t = unit; t < num_tiles && ok; t += num_units, ++tile_i) {
                    int problem = 0, tm, tn;
                    if constexpr (BATCHED) tile_coords_batched(t, p, problem, tm, tn);
                    else tile_coords(t, p, tm, tn);
                    const int row_a = (tm * kCtas + (int)rank) * kBlockM;
                    const int row_b = tn * BN + (TWO_SM ? (int)rank * (BN / 2) : 0);
                    if (pacing && tile_i > 0) {
                        // Pacing, not a dependency: CTAs that drift apart stop finding each other's A / B panels in
                        // L2 (they are re-read from DRAM instead).  Wait, for at most ~20 us, until most CTAs have
                        // finished loading the previous round of tiles.
                        const int target = (int)(((int64_t)tile_i * num_units * p.pace_pct) / 100);
                        const long long t0 = clock64();
                        bool in_time = true;
                        while (*(volatile int*)p.pace < target && (in_time = (clock64() - t0 < 40000))) { }
                        if (!in_time) pacing = false;      // the other CTAs are not running alongside: stop waiting for them
                    }
                    for (int kb = 0; kb < num_kb; ++kb) {
                        if (!mbar_wait(empty_bar(s), ph ^ 1u, wctx, SITE_PRODUCER_EMPTY, kb)) { ok = false; break; }
                        const uint32_t sa = smem_base + s * Plan::kStageBytes;
                        const uint32_t sb = sa + Plan::kABytes;
                        if constexpr (TWO_SM) {
                            if (leader) mbar_arrive_expect_tx(full_bar(s), 2u * Plan::kStageBytes);
                        } else {
                            mbar_arrive_expect_tx(full_bar(s), (uint32_t)Plan::kStageBytes);
                        }
                        load_stage<KIND, TWO_SM, BN, A_MN, B_MN, BATCHED>(&map_a, &map_b, sa, sb, full_bar(s), kb, row_a, row_b,
                                                                          problem, p.a_batched, p.b_batched, pol_a, pol_b);
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                    if (p.pace_pct > 0 && leader && ok) atomicAdd(p.pace, 1);   // counted even after this CTA stopped waiting
                }
                if (!ok) record_give_up();
            };
            using T = std::true_type;
            using F = std::false_type;
            if (p.batch == 1) {
                if (layout == 0) produce(F{}, F{}, F{});
                else if (layout == 1) produce(T{}, F{}, F{});
                else if constexpr (kBMnOk) {
                    if (layout == 2) produce(F{}, T{}, F{});
                    else produce(T{}, T{}, F{});
                }
            } else {
                if (layout == 0) produce(F{}, F{}, T{});
                else if (layout == 1) produce(T{}, F{}, T{});
                else if constexpr (kBMnOk) {
                    if (layout == 2) produce(F{}, T{}, T{});
                    else produce(T{}, T{}, T{});
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (rank 0 of a pair only) ----------------
        if (lane == 0 && leader) {
            // as for the producer: one instantiation of the loop per operand layout, chosen once
            auto issue = [&](auto a_mn_tag, auto b_mn_tag) {
                constexpr bool A_MN = decltype(a_mn_tag)::value, B_MN = decltype(b_mn_tag)::value;
                int s = 0;
                uint32_t ph = 0;
                int local = 0;
                bool ok = true;
                for (int t = unit; t < num_tiles && ok; t += num_units, ++local) {
                    const int buf = local & 1;
                    const uint32_t tph = (local >> 1) & 1u;
                    if (!mbar_wait(tmem_empty_bar(buf), tph ^ 1u, wctx, SITE_MMA_TMEM_EMPTY, local)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                    for (int kb = 0; kb < num_kb; ++kb) {
                        if (!mbar_wait(full_bar(s), ph, wctx, SITE_MMA_FULL, kb)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t sa = smem_base + s * Plan::kStageBytes;
                        const uint32_t sb = sa + Plan::kABytes;
                        issue_stage<KIND, TWO_SM, A_MN, B_MN>(tmem_d, sa, sb, p.idesc, kb == 0);
                        umma_commit<TWO_SM>(empty_bar(s));            // frees the stage once these MMAs have read it
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                    // accumulator complete (the time-out self-test leaves out the one that completes this CTA's last tile:
                    // its MMAs still finish, but nothing tells the epilogue, whose bounded wait then runs out)
                    if (ok && !(p.drop_commit && t + num_units >= num_tiles)) umma_commit<TWO_SM>(tmem_full_bar(buf));
                }
                if (!ok) record_give_up();
            };
            if (layout == 0) issue(std::false_type{}, std::false_type{});
            else if (layout == 1) issue(std::true_type{}, std::false_type{});
            else if (layout == 2) issue(std::false_type{}, std::true_type{});
            else issue(std::true_type{}, std::true_type{});
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int q = warp & 3;                       // TMEM lane quarter this warp may access
        const bool c_vec = (p.cs1 == 1) && ((p.cs0 * (int64_t)sizeof(TC)) % 16 == 0) &&
                           ((p.c_bs * (int64_t)sizeof(TC)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        int local = 0;
        bool ok = true;
        uint32_t store_count = 0;                    // TMA-store boxes this warp has issued (warp-uniform)
        const int ew = warp - 2;                      // epilogue warp 0 .. epi_warps - 1
        const int half = ew >> 2;                     // eight warps: warps 4 .. 7 take the second half of the tile's columns
        const uint32_t n_boxes = (uint32_t)(p.c_in ? cin_boxes : base_boxes);  // staging boxes of this warp
        uint8_t* store_stage = smem_gen + S * Plan::kStageBytes + (size_t)ew * n_boxes * Plan::kStoreBoxBytes;
        // c_in: the old C of every box this warp will produce is copied (cp.async, 16 bytes per lane, 8 lanes per
        // 128-byte row, swizzled like the box) into the staging box the result is later written to, in the order in
        // which the boxes are produced and as far ahead as the ring allows - the first boxes of the next tile while
        // this warp still waits for that tile's accumulator.  The n-th copy and the n-th result use box n % n_boxes.
        constexpr int kBoxCols = 128 / (int)sizeof(TC);          // columns per staging box
        constexpr int kPerVec = 16 / (int)sizeof(TC);
        const int vu = lane & 7, vr4 = lane >> 3;                // this lane's 16-byte unit and row (mod 4) in box moves
        uint32_t cin_issued = 0;                     // boxes whose copy has been issued (warp-uniform)
        int cin_t = unit, cin_box = 0;               // the tile and the box in it that is copied next
        int64_t cin_row0 = 0, cin_col_tile = 0;
        const TC* cin_c = C;                         // C of the problem the copied tile belongs to
        auto cin_issue_upto = [&](uint32_t limit) {
            while (cin_issued < limit && cin_t < num_tiles) {
                if (cin_box == 0) {
                    int problem, tm, tn;
                    tile_coords_batched(cin_t, p, problem, tm, tn);
                    cin_row0 = (int64_t)(tm * kCtas + (int)rank) * kBlockM + q * 32;
                    cin_col_tile = (int64_t)tn * BN;
                    cin_c = C + (int64_t)problem * p.c_bs;
                }
                const int64_t box_col0 = cin_col_tile + (int64_t)(half * boxes_per_warp_tile + cin_box) * kBoxCols;
                if (cin_row0 < p.m && box_col0 < p.n) {
                    uint8_t* dst_box = store_stage + (size_t)(cin_issued % n_boxes) * Plan::kStoreBoxBytes;
                    const int64_t col = box_col0 + (int64_t)vu * kPerVec;
                    const bool col_ok = col + kPerVec <= p.n;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = 4 * i + vr4;
                        uint8_t* dst = dst_box + r * 128 + ((vu ^ (r & 7)) << 4);
                        if (col_ok && cin_row0 + r < p.m)
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(cin_c + (cin_row0 + r) * p.cs0 + col) : "memory");
                        else
                            *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);    // outside the matrix: never stored
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    ++cin_issued;
                }
                if (++cin_box == boxes_per_warp_tile) { cin_box = 0; cin_t += num_units; }
            }
        };
        if (p.c_in) cin_issue_upto(n_boxes);
        for (int t = unit; t < num_tiles && ok; t += num_units, ++local) {
            int problem, tm, tn;
            tile_coords_batched(t, p, problem, tm, tn);
            const int buf = local & 1;
            const uint32_t tph = (local >> 1) & 1u;
            // all 32 lanes must agree before the warp-wide TMEM loads below
            if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), tph, wctx, SITE_EPI_TMEM_FULL, local))) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t row = (int64_t)(tm * kCtas + (int)rank) * kBlockM + q * 32 + lane;
            const int64_t col_tile = (int64_t)tn * BN;
            TC* crow = C + (int64_t)problem * p.c_bs + row * p.cs0;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            const int64_t row0 = (int64_t)(tm * kCtas + (int)rank) * kBlockM + q * 32;     // first row of this warp
            auto process_chunk = [&](int c, const uint32_t (&acc)[32]) {
                const int64_t col0 = col_tile + c * 32;
                if (!p.tma_store && !p.lsu_stage) {
                    if (row < p.m && col0 < p.n) {
                        const int ncols = (int)min((int64_t)32, p.n - col0);
                        epilogue_row<TC, ACC>(acc, crow, col0, ncols, c_vec, p.cs1, bias, p);
                    }
                } else {
                    // a staging box is 128 bytes wide: one 32-column chunk of 4-byte results, two of 2-byte ones
                    constexpr int CPB = (sizeof(TC) == 4) ? 1 : 2;
                    const int sub = c % CPB;
                    const int64_t box_col0 = col0 - (int64_t)sub * 32;
                    const bool box_live = (row0 < p.m) && (box_col0 < p.n);      // warp-uniform
                    uint8_t* box = store_stage + (size_t)(store_count % n_boxes) * Plan::kStoreBoxBytes;
                    if (p.c_in) {
                        if (box_live && sub == 0) {
                            // the old C of this box was requested boxes ago: wait for this lane's part of it, leaving the
                            // copies of the boxes after it in flight, then for the other lanes' parts
                            switch (cin_issued - 1u - store_count) {
                            case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
                            case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
                            case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
                            default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
                            }
                            __syncwarp();
                        }
                        if (box_live && col0 < p.n) {
                            const int ncols = (int)min((int64_t)32, p.n - col0);
                            epilogue_inplace<TC, ACC>(acc, col0, ncols, bias, p, box + lane * 128, sub * (32 * (int)sizeof(TC) / 16), lane & 7);
                        }
                    } else {
                        if (box_live && sub == 0 && store_count >= 2 && !p.lsu_stage) {
                            // the box about to be overwritten was handed to TMA two boxes ago: wait until it has been read
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                            __syncwarp();
                        }
                        if (box_live && col0 < p.n) {
                            const int ncols = (int)min((int64_t)32, p.n - col0);
                            epilogue_to_smem<TC, ACC>(acc, crow, row < p.m, col0, ncols, c_vec, bias, p, box + lane * 128,
                                                      sub * (32 * (int)sizeof(TC) / 16), lane & 7);
                        }
                    }
                    if (box_live && sub == CPB - 1 && p.lsu_stage) {
                        // the warp moves the finished box to C itself: 8 lanes per 128-byte row, 4 rows per step
                        __syncwarp();
                        const int64_t col = box_col0 + (int64_t)vu * kPerVec;
                        const bool col_ok = col + kPerVec <= p.n;
                        uint4 v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = 4 * i + vr4;
                            v[i] = *reinterpret_cast<const uint4*>(box + r * 128 + ((vu ^ (r & 7)) << 4));
                        }
                        TC* dst = C + (int64_t)problem * p.c_bs + (row0 + vr4) * p.cs0 + col;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (col_ok && row0 + 4 * i + vr4 < p.m) *reinterpret_cast<uint4*>(dst + (int64_t)(4 * i) * p.cs0) = v[i];
                        __syncwarp();                // the box may be written again
                        ++store_count;
                        if (p.c_in) cin_issue_upto(store_count + n_boxes);
                    } else if (box_live && sub == CPB - 1) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to TMA
                        __syncwarp();
                        if (lane == 0) {
                            const uint32_t src = smem_u32(box);
                            const int n_tma = (p.peer_store || p.copy_ctas > 0) ? 1 : p.n_replicas;
                            for (int r = 0; r < n_tma; ++r) tma_store_2d(&cmaps.m[r], src, (int)box_col0, (int)row0);
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                        if (p.peer_store && p.copy_ctas == 0 && p.n_replicas > 1) {
                            // Replicas in other GPUs' memory: the warp reads the box back, 16 bytes per lane (8 lanes
                            // cover one 128-byte row, a step covers 4 rows), and writes it to every peer with plain
                            // stores.  A TMA store that waits for NVLink holds up the operand loads queued behind it in
                            // the same TMA unit; these stores wait in the load/store path instead.
                            const int u = lane & 7, r4 = lane >> 3;
                            constexpr int kPerVec = 16 / (int)sizeof(TC);
                            const int64_t colu = box_col0 + (int64_t)u * kPerVec;
                            const bool col_ok = colu + kPerVec <= p.n;
                            uint4 v[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int r = 4 * i + r4;
                                v[i] = *reinterpret_cast<const uint4*>(box + r * 128 + ((u ^ (r & 7)) << 4));
                            }
                            const int64_t row_step = 4 * p.cs0 * (int64_t)sizeof(TC);
                            for (int rep = 1; rep < p.n_replicas; ++rep) {
                                char* dst = reinterpret_cast<char*>(p.peer_c[rep - 1]) +
                                            ((row0 + r4) * p.cs0 + colu) * (int64_t)sizeof(TC);
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (col_ok && row0 + 4 * i + r4 < p.m) *reinterpret_cast<uint4*>(dst + i * row_step) = v[i];
                            }
                        }
                        ++store_count;
                    }
                }
            };
            // this warp's share of the accumulator, 32 columns at a time
            {
                const int per_half = (BN / 32) / halves;
#pragma unroll 1
                for (int c = half * per_half; c < (half + 1) * per_half; ++c) {
                    uint32_t acc[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), acc);
                    tmem_wait_ld(acc);
                    process_chunk(c, acc);
                }
            }
            // this warp has drained its part of the accumulator: hand it back to the MMA issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(TWO_SM ? (tmem_empty_bar(buf) & kPeerMask) : tmem_empty_bar(buf));
            if (p.copy_ctas > 0 && lane == 0) {
                // this warp's part of the tile is on its way to C: once the stores have completed, publish it to
                // the forwarding CTAs (TMA writes belong to the async proxy, the readers use ordinary loads)
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __threadfence();
                asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.tile_flags + t) : "memory");
            }
        }
        if (!ok && lane == 0) record_give_up();
        // Before the CTA exits its TMA stores must at least have read their shared-memory boxes; the global writes
        // themselves are complete when the grid is.  Stores into other GPUs' memory are waited for in full.
        if (lane == 0) {
            if (p.n_replicas > 1 && p.copy_ctas == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
        __syncwarp();
    }

    // teardown: every role ends here, also after a bounded wait gave up
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (TWO_SM) cluster_sync_all(); else __syncthreads();
    if ((gave_up[0] | gave_up[1]) != 0u) {
        // failure path: give loads that are still in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if constexpr (TWO_SM) cluster_sync_all(); else __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (TWO_SM)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    // resolved through the runtime so that the library has no link-time dependency on the driver library
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}

int elem_size(int t)
{
    switch (t) {
    case ACCB_F32: case ACCB_S32: return 4;
    case ACCB_F16: case ACCB_BF16: case ACCB_S16: return 2;
    default: return 1;
    }
}

// K-major operand [rows, k] with `ld` elements between rows; box = 128 bytes of K by box_rows rows
bool make_operand_map(CUtensorMap* map, const void* base, int type, int64_t rows, int64_t k, int64_t ld, int box_rows,
                      bool mn_major = false, int64_t batch = 1, int64_t batch_stride = 0)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    CUtensorMapDataType dt;
    switch (type) {
    case ACCB_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case ACCB_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case ACCB_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    }
    const int es = elem_size(type);
    // K-major: [rows][k], k contiguous, box = 128 bytes of k by box_rows rows.
    // MN-major: the array is [k][rows] with `rows` (M or N) contiguous; box = 128 bytes of M/N by (128 / es) k-rows.
    // Batched (batch > 1 with a non-zero batch stride): a third, outermost dimension walks the problems; the box
    // is one problem thick, so it lands in shared memory exactly like the rank-2 box.
    const bool rank3 = batch > 1 && batch_stride > 0;
    cuuint64_t dims[3] = { (cuuint64_t)(mn_major ? rows : k), (cuuint64_t)(mn_major ? k : rows), (cuuint64_t)batch };
    cuuint64_t strides[2] = { (cuuint64_t)(ld * es), (cuuint64_t)(batch_stride * es) };
    cuuint32_t box[3] = { (cuuint32_t)(kSlabBytes / es), (cuuint32_t)(mn_major ? kSlabBytes / es : box_rows), 1 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = enc(map, dt, rank3 ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// C (or a replica of it) as a row-major [m, n] tensor; box = 32 rows of 128 bytes, 128-byte swizzle
bool make_c_map(CUtensorMap* map, void* base, int type, int64_t m, int64_t n, int64_t ld)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    CUtensorMapDataType dt;
    switch (type) {
    case ACCB_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case ACCB_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case ACCB_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_INT32; break;
    }
    const int es = elem_size(type);
    cuuint64_t dims[2] = { (cuuint64_t)n, (cuuint64_t)m };
    cuuint64_t strides[1] = { (cuuint64_t)(ld * es) };
    cuuint32_t box[2] = { (cuuint32_t)(128 / es), 32 };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = enc(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool c_tma_storable(const accb_gemm_desc& d, const void* c)
{
    return d.c_stride[1] == 1 && (d.c_stride[0] * elem_size(d.c_type)) % 16 == 0 &&
           (reinterpret_cast<uintptr_t>(c) & 15) == 0;
}

// Launches whose epilogue shows - a K loop of up to 32 slabs of 128 bytes (K = 2048 for 16-bit operands), or up to 64
// when every CTA has one tile only, so that nothing overlaps its epilogue - and whose C can be moved box by box
// (row-major, 16-byte aligned rows and row ends, one problem, no replicas) take the epilogue with warp-moved boxes and
// eight epilogue warps.
bool short_k_epilogue(const GemmLaunch& g, bool one_round)
{
    const accb_gemm_desc& d = g.d;
    const int64_t slabs = (d.k * elem_size(d.a_type) + kSlabBytes - 1) / kSlabBytes;
    const bool c_ok = d.c_stride[1] == 1 && (d.c_stride[0] * elem_size(d.c_type)) % 16 == 0 &&
                      (reinterpret_cast<uintptr_t>(g.c) & 15) == 0 && ((d.n * elem_size(d.c_type)) % 16) == 0;
    const bool batch_ok = g.batch <= 1 || (g.c_batch_stride * elem_size(d.c_type)) % 16 == 0;
    return c_ok && batch_ok && g.n_extra_c == 0 && (slabs <= 32 || (one_round && slabs <= 64));
}

uint32_t make_idesc(int a_type, int b_type, bool int_acc, bool f16_out_acc, int m, int n, bool a_mn = false, bool b_mn = false)
{
    auto fmt = [](int t) -> uint32_t {
        switch (t) {
        case ACCB_F16: return 0; case ACCB_BF16: return 1; case ACCB_F32: return 2;   // f16, bf16, tf32
        case ACCB_S8: return 1; default: return 0;                                    // s8, u8
        }
    };
    uint32_t d = 0;
    d |= (int_acc ? 2u : (f16_out_acc ? 0u : 1u)) << 4;   // accumulator format: s32 / f16 / f32
    d |= fmt(a_type) << 7;
    d |= fmt(b_type) << 10;
    // bits 13, 14: no negation; bits 15, 16: operand major-ness (0 = K-major, 1 = MN-major)
    d |= (a_mn ? 1u : 0u) << 15;
    d |= (b_mn ? 1u : 0u) << 16;
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(m >> 4) << 24;
    return d;
}

template <int KIND, typename TC, bool TWO_SM, int BN>
int launch_variant(const GemmLaunch& g, const CUtensorMap& ma, const CUtensorMap& mb, const CReplicaMaps& cm, UmmaParams p,
                   const char** err)
{
    using Plan = SmemPlan<TWO_SM, BN>;
    auto kernel = gemm_umma_kernel<KIND, TC, TWO_SM, BN>;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(32u * (2u + (unsigned)p.epi_warps));
    cfg.dynamicSmemBytes = Plan::kTotal;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (TWO_SM) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
        attr[cfg.numAttrs].val.clusterDim.x = 2; attr[cfg.numAttrs].val.clusterDim.y = 1; attr[cfg.numAttrs].val.clusterDim.z = 1;
        ++cfg.numAttrs;
    }
    if (p.pdl) {
        // let this launch be scheduled while the previous kernel of the stream is still running (see the kernel's
        // griddepcontrol.wait): hides the launch and the set-up of back-to-back GEMMs
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        ++cfg.numAttrs;
    }
    // Per device and kernel variant, once: opt in to the large dynamic shared memory and find how many CTAs
    // (pairs) can be resident.  Both calls cost microseconds, which is the whole run time of a small GEMM.
    constexpr int kMaxDevices = 64;
    static std::atomic<int> resident_units[kMaxDevices];
    const int slot = (g.device >= 0 && g.device < kMaxDevices) ? g.device : -1;
    int units = slot >= 0 ? resident_units[slot].load(std::memory_order_acquire) : 0;
    if (units == 0) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kTotal);
        if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
        units = g.num_sms;
        if (TWO_SM) {
            cfg.gridDim = dim3(2 * (unsigned)(g.num_sms / 2));
            int max_clusters = 0;
            e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg);
            if (e != cudaSuccess || max_clusters < 1) { *err = "tcgen05 GEMM: no CTA pair can be resident"; (void)cudaGetLastError(); return ACCB_ERR_CUDA; }
            units = max_clusters < g.num_sms / 2 ? max_clusters : g.num_sms / 2;
        }
        if (slot >= 0) resident_units[slot].store(units, std::memory_order_release);
    }
    const int num_tiles = p.tiles_m * p.tiles_n * p.batch;
    if (g.d.max_ctas > 0) {
        const int cap = g.d.max_ctas / (TWO_SM ? 2 : 1);
        if (cap >= 1 && cap < units) units = cap;
    }
    // forwarding CTAs take whole units (clusters) out of the resident set; the rest compute
    const int copy_units = p.copy_ctas / (TWO_SM ? 2 : 1);
    if (copy_units > 0) {
        if (units - copy_units < 1) { *err = "tcgen05 GEMM: no SM left for computing beside the forwarding CTAs"; return ACCB_ERR_ARG; }
        units -= copy_units;
    }
    if (units > num_tiles) units = num_tiles;
    if (p.verbose)
        fprintf(stderr, "tcgen05 GEMM %lld x %lld x %lld x %d: %s tiles of %d columns, %d tiles on %d %s, pacing %d%%\n",
                (long long)p.m, (long long)p.n, (long long)p.k, p.batch, TWO_SM ? "pair" : "single-CTA", BN, num_tiles, units,
                TWO_SM ? "pairs" : "CTAs", p.pace_pct);
    if (p.verbose && p.lsu_stage) fprintf(stderr, "  staged epilogue without TMA%s, %d operand stages\n", p.c_in ? ", old C copied in boxes ahead" : "", (p.c_in && BN * (int)sizeof(TC) / 128 > 2) ? Plan::kCinStages : Plan::kStages);
    if (p.verbose) fprintf(stderr, "  %d epilogue warps\n", p.epi_warps);
    if (p.verbose && p.n_replicas > 1)
        fprintf(stderr, "  %d replicas: %s\n", p.n_replicas, p.copy_ctas > 0 ? "forwarding CTAs" : p.peer_store ? "register stores from the epilogue" : "TMA stores from the epilogue");
    cfg.gridDim = dim3((unsigned)((units + copy_units) * (TWO_SM ? 2 : 1)));
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mb, cm, (TC*)g.c, g.bias, p);
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
    note_launches(1);
    return 1;
}

// Tile shape for one problem: CTA pairs (256-row tiles) or single CTAs (128 rows), 256 or 128 columns.
// The kernel is persistent, so its run time is (rounds of tiles) x (time of one tile) plus the last tile's
// epilogue, which nothing overlaps.  A wide pair tile is the most efficient per flop, but a problem whose
// tile count is just over a multiple of the resident CTAs wastes most of a round; a narrower tile then wins.
struct TileChoice { bool two_sm; int bn; };

TileChoice choose_tile(const GemmLaunch& g, int want_two_sm /* -1: free, 0 / 1: fixed by the caller */)
{
    const accb_gemm_desc& d = g.d;
    const int64_t batch = g.batch > 1 ? g.batch : 1;
    const bool b_mn = d.b_stride[0] != 1;
    const bool eight_bit = elem_size(d.a_type) == 1;
    // throughput of each tile shape on a large square bf16 problem relative to the 256-column pair tile (measured:
    // 1518 / 1346 / 972 / 851 TFLOP/s at 8192^3).  128-column tiles need 1.5x the L2 -> shared-memory traffic
    // per flop and are bound by it; they only pay on problems too small to give every SM a 256-column tile.
    static const double kEff[2][2] = { /* 1 SM */ { 0.64 /*128*/, 0.89 /*256*/ }, /* pair */ { 0.56 /*128*/, 1.00 /*256*/ } };
    const int force_bn = g.force_tile_cols ? g.force_tile_cols : options().gemm_tile_cols;
    TileChoice best{want_two_sm != 0, kBlockN};
    double best_cost = -1.0;
    for (int two = 1; two >= 0; --two) {
        if (want_two_sm >= 0 && two != want_two_sm) continue;
        for (int bn = 256; bn >= 128; bn -= 128) {
            if (force_bn && bn != force_bn) continue;
            if (two && bn == 128 && eight_bit && b_mn) continue;      // a 64-column share of B is narrower than one box
            const int64_t rows = two ? 2 * kBlockM : kBlockM;
            const int64_t tiles = ((d.m + rows - 1) / rows) * ((d.n + bn - 1) / bn) * batch;
            int64_t units = two ? g.num_sms / 2 : g.num_sms;
            if (d.max_ctas > 0 && d.max_ctas / (two ? 2 : 1) >= 1 && d.max_ctas / (two ? 2 : 1) < units) units = d.max_ctas / (two ? 2 : 1);
            const int64_t rounds = (tiles + units - 1) / units;
            const double k_steps = (double)((d.k + 63) / 64);
            // per tile: K loop + (only for the last round) the epilogue, both proportional to the tile's columns
            const double cost = ((double)rounds * k_steps + 6.0) * bn / kEff[two][bn == 256];
            if (best_cost < 0.0 || cost < best_cost * 0.97) { best_cost = cost; best = TileChoice{two != 0, bn}; }
        }
    }
    return best;
}

}  // namespace

void gemm_umma_tile_plan(const GemmLaunch& g, int want_two_sm, int* two_sm, int* tile_cols, int64_t* tiles, int64_t* rounds)
{
    const TileChoice t = choose_tile(g, want_two_sm);
    const int64_t rows = t.two_sm ? 2 * kBlockM : kBlockM;
    const int64_t batch = g.batch > 1 ? g.batch : 1;
    const int64_t n_tiles = ((g.d.m + rows - 1) / rows) * ((g.d.n + t.bn - 1) / t.bn) * batch;
    int64_t units = t.two_sm ? g.num_sms / 2 : g.num_sms;
    if (g.d.max_ctas > 0 && g.d.max_ctas / (t.two_sm ? 2 : 1) >= 1 && g.d.max_ctas / (t.two_sm ? 2 : 1) < units)
        units = g.d.max_ctas / (t.two_sm ? 2 : 1);
    if (units < 1) units = 1;
    *two_sm = t.two_sm ? 1 : 0;
    *tile_cols = t.bn;
    *tiles = n_tiles;
    *rounds = (n_tiles + units - 1) / units;
}

void gemm_umma_launch_geometry(const GemmLaunch& g, int want_two_sm, int32_t out[8])
{
    const TileChoice t = choose_tile(g, want_two_sm);
    const int64_t rows = t.two_sm ? 2 * kBlockM : kBlockM;
    const int64_t batch = g.batch > 1 ? g.batch : 1;
    const int64_t n_tiles = ((g.d.m + rows - 1) / rows) * ((g.d.n + t.bn - 1) / t.bn) * batch;
    const int per = t.two_sm ? 2 : 1;
    int64_t units = g.num_sms / per;
    if (g.d.max_ctas > 0 && g.d.max_ctas / per >= 1 && g.d.max_ctas / per < units) units = g.d.max_ctas / per;
    const bool one_round = n_tiles <= units;
    if (units > n_tiles) units = n_tiles;
    if (units < 1) units = 1;
    int smem = 0, stages = 0;
    if (t.two_sm) {
        if (t.bn == 256) { smem = SmemPlan<true, 256>::kTotal; stages = SmemPlan<true, 256>::kStages; }
        else { smem = SmemPlan<true, 128>::kTotal; stages = SmemPlan<true, 128>::kStages; }
    } else {
        if (t.bn == 256) { smem = SmemPlan<false, 256>::kTotal; stages = SmemPlan<false, 256>::kStages; }
        else { smem = SmemPlan<false, 128>::kTotal; stages = SmemPlan<false, 128>::kStages; }
    }
    out[0] = (int32_t)(units * per); out[1] = 1; out[2] = 1;
    out[3] = short_k_epilogue(g, one_round) ? kThreadsWide : kThreads; out[4] = 1; out[5] = 1;
    out[6] = smem;
    out[7] = stages;
}

bool gemm_umma_types_supported(const accb_gemm_desc& d)
{
    const int a = d.a_type, b = d.b_type, c = d.c_type;
    const bool f16_family = (a == ACCB_F16 && b == ACCB_F16 && (c == ACCB_F32 || c == ACCB_F16)) ||
                            (a == ACCB_BF16 && b == ACCB_BF16 && (c == ACCB_F32 || c == ACCB_BF16));
    const bool tf32 = (a == ACCB_F32 && b == ACCB_F32 && c == ACCB_F32);
    const bool i8 = ((a == ACCB_S8 || a == ACCB_U8) && (b == ACCB_S8 || b == ACCB_U8) && c == ACCB_S32);
    return f16_family || tf32 || i8;
}

bool gemm_umma_supported(const GemmLaunch& g, const char** why)
{
    const accb_gemm_desc& d = g.d;
    const int a = d.a_type, b = d.b_type, c = d.c_type;
    const bool tf32 = (a == ACCB_F32 && b == ACCB_F32 && c == ACCB_F32);
    const bool i8 = ((a == ACCB_S8 || a == ACCB_U8) && (b == ACCB_S8 || b == ACCB_U8) && c == ACCB_S32);
    if (!gemm_umma_types_supported(d)) { *why = "element types have no tensor-core path"; return false; }
    if (i8 && (d.alpha != 1.0f || (d.beta != 0.0f && d.beta != 1.0f) || g.bias)) { *why = "integer GEMM supports alpha=1, beta in {0,1}, no bias"; return false; }
    // each operand must be contiguous along K (row-major A / column-major B) or along M / N (column-major A /
    // row-major B); the other stride is the pitch
    const bool a_k = d.a_stride[1] == 1, a_mn = !a_k && d.a_stride[0] == 1;
    const bool b_k = d.b_stride[0] == 1, b_mn = !b_k && d.b_stride[1] == 1;
    if (!(a_k || a_mn) || !(b_k || b_mn)) { *why = "tensor-core path needs unit stride along one dimension of A and of B"; return false; }
    // 32-bit (TF32) operands are taken K-contiguous only: their M / N-contiguous form needs a different
    // shared-memory swizzle (32-byte base atom) that this kernel does not stage
    if (tf32 && (a_mn || b_mn)) { *why = "TF32 tensor path needs K-contiguous A (row-major) and B (column-major)"; return false; }
    const int es = elem_size(a);
    const int64_t pitch_a = a_k ? d.a_stride[0] : d.a_stride[1], pitch_b = b_k ? d.b_stride[1] : d.b_stride[0];
    if ((pitch_a * es) % 16 || (pitch_b * es) % 16) { *why = "operand row pitch must be a multiple of 16 bytes"; return false; }
    if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15)) { *why = "operand base must be 16-byte aligned"; return false; }
    if (g.batch > 1) {
        if (g.n_extra_c > 0) { *why = "C replicas are not available for batched GEMMs"; return false; }
        if (g.a_batch_stride < 0 || g.b_batch_stride < 0 || g.c_batch_stride < 0) { *why = "batch strides must not be negative"; return false; }
        if ((g.a_batch_stride * es) % 16 || (g.b_batch_stride * es) % 16) { *why = "operand batch stride must be a multiple of 16 bytes"; return false; }
        if (g.batch > (1 << 20)) { *why = "too many problems in one batched call"; return false; }
    }
    if (d.m < 1 || d.n < 1 || d.k < 1) { *why = "empty problem"; return false; }
    if (d.m > (int64_t)1 << 30 || d.n > (int64_t)1 << 30 || d.k > (int64_t)1 << 30) { *why = "dimension too large"; return false; }
    if (!encode_tiled_fn()) { *why = "cuTensorMapEncodeTiled is not available"; return false; }
    return true;
}

int launch_gemm_umma(const GemmLaunch& g, int want_two_sm, const char** err)
{
    const accb_gemm_desc& d = g.d;
    const char* why = nullptr;
    if (!gemm_umma_supported(g, &why)) { *err = why; return ACCB_ERR_ARG; }

    const TileChoice tile = choose_tile(g, want_two_sm);
    const bool two_sm = tile.two_sm;
    const int bn = tile.bn;
    CUtensorMap ma, mb;
    const int b_box_rows = two_sm ? bn / 2 : bn;
    const bool a_mn = d.a_stride[1] != 1, b_mn = d.b_stride[0] != 1;
    const int64_t batch = g.batch > 1 ? g.batch : 1;
    if (!make_operand_map(&ma, g.a, d.a_type, d.m, d.k, a_mn ? d.a_stride[1] : d.a_stride[0], kBlockM, a_mn, batch, g.a_batch_stride) ||
        !make_operand_map(&mb, g.b, d.b_type, d.n, d.k, b_mn ? d.b_stride[0] : d.b_stride[1], b_box_rows, b_mn, batch, g.b_batch_stride)) {
        *err = "tcgen05 GEMM: cuTensorMapEncodeTiled failed";
        return ACCB_ERR_CUDA;
    }

    const bool int_acc = (d.c_type == ACCB_S32);
    UmmaParams p;
    memset(&p, 0, sizeof p);
    p.m = d.m; p.n = d.n; p.k = d.k;
    p.cs0 = d.c_stride[0]; p.cs1 = d.c_stride[1];
    p.alpha = d.alpha; p.beta = d.beta; p.relu = (d.epilogue == ACCB_EPI_RELU);
    p.idesc = make_idesc(d.a_type, d.b_type, int_acc, false, two_sm ? 2 * kBlockM : kBlockM, bn, a_mn, b_mn);
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.elem_bytes = elem_size(d.a_type);
    const int rows_per_unit = two_sm ? 2 * kBlockM : kBlockM;
    p.tiles_m = (int)((d.m + rows_per_unit - 1) / rows_per_unit);
    p.tiles_n = (int)((d.n + bn - 1) / bn);
    p.group_m = two_sm ? 8 : 16;
    p.batch = (int)batch;
    p.a_batched = (batch > 1 && g.a_batch_stride > 0) ? 1 : 0;
    p.b_batched = (batch > 1 && g.b_batch_stride > 0) ? 1 : 0;
    p.c_bs = batch > 1 ? g.c_batch_stride : 0;
    const int64_t tiles_total = (int64_t)p.tiles_m * p.tiles_n * batch;
    const int64_t units_est = two_sm ? g.num_sms / 2 : g.num_sms;
    // Epilogue path: staged TMA stores whenever C allows it.  Storing straight from registers looked 2 - 3 us
    // faster for one-round problems when each launch was timed cold under a profiler, but is equal or slower
    // (4096 x 768 x 3072: 784 vs 852 TFLOP/s) in a warm launch sequence.  Batched problems use plain stores.
    p.tma_store = (c_tma_storable(d, g.c) && batch == 1) ? 1 : 0;
    p.n_replicas = 1 + g.n_extra_c;
    // Long launches: keep the persistent CTAs in step tile by tile.  Left alone they drift apart over a hundred
    // rounds of tiles and stop sharing A / B panels in L2 (measured on 65536 x 8192 x 8192: 22.8 GB of DRAM
    // traffic per launch without pacing, about 11 GB with it).  Short launches do not drift far enough to matter.
    p.pace_pct = (tiles_total >= 8 * units_est) ? 100 : 0;
    if (p.pace_pct && two_sm && p.tiles_m >= 32) p.group_m = 16;
    p.pace = g.status + kStatusWords;
    {
        // per-thread overrides (accb_set_option): tests reach every path on small problems with them
        const Options& o = options();
        if (o.gemm_group_m > 0) p.group_m = o.gemm_group_m;
        p.hint_a = o.gemm_hint_a; p.hint_b = o.gemm_hint_b; p.c_stream = o.gemm_c_stream;
        if (o.gemm_staged_store >= 0 && g.n_extra_c == 0) p.tma_store = (o.gemm_staged_store && c_tma_storable(d, g.c) && batch == 1) ? 1 : 0;
        if (o.gemm_pace_pct >= 0) p.pace_pct = o.gemm_pace_pct;
        p.verbose = o.gemm_verbose;
        p.wait_ns = o.gemm_wait_limit_us > 0 ? (unsigned long long)o.gemm_wait_limit_us * 1000ull : 1000000000ull;
        p.drop_commit = o.gemm_test_drop_commit ? 1 : 0;
        p.pdl = o.gemm_pdl < 0 ? 1 : (o.gemm_pdl ? 1 : 0);
        // peers are written with register stores unless the caller asks for TMA stores or a row's last vector is partial
        const bool vec_rows = ((d.n * elem_size(d.c_type)) % 16) == 0;
        p.peer_store = (g.n_extra_c > 0 && vec_rows && (o.gemm_peer_store < 0 ? kPeerStoreDefault : o.gemm_peer_store)) ? 1 : 0;
    }
    p.launch_id = g.launch_id;
    // A short K loop (up to 32 slabs of 128 bytes: K = 2048 for 16-bit operands): the epilogue of a CTA's last tile is a
    // large part of the launch, and with several tiles per CTA the epilogue, not the K loop, sets the pace.  Timestamps
    // inside the kernel (1024^3 bf16, C += A @ B: 1.5 us from the start to the first operands, 4.6 us of K loop, 2.6 us
    // of epilogue for 128 columns) show an epilogue warp, alone on its scheduler, bound by instruction latency.  Such
    // launches get eight epilogue warps, two per TMEM lane quarter, each taking half of the tile's columns; the warps
    // move their staging boxes to C themselves and, with beta != 0, copy the old C into them boxes ahead (the first
    // boxes of a tile while its K loop still runs) instead of reading it row by row when it is needed; for tiles wider
    // than the boxes every launch has, the extra boxes cost the operand ring one stage.  Measured, C += A @ B in bf16,
    // against the first epilogue (four warps, TMA-stored boxes): 1024^3 9.9 against 12.0 us, 2048^3 18.1 / 23.0,
    // 3072 x 2048 x 1024 18.0 / 26.1, 4096 x 4096 x 1024 37.1 / 45.5 (fp32 results 40.3 / 68.9); with beta = 0
    // 4096 x 4096 x 1024 28.7 / 32.7.  At K = 4096 it is equal or slower (4096^3 120 / 119) and 2 % slower at
    // 65536 x 8192 x 8192, which is why long K loops keep four warps and the TMA stores.
    {
        const Options& o = options();
        const int per = two_sm ? 2 : 1;
        const int64_t units_cap = (d.max_ctas > 0 && d.max_ctas / per >= 1 && d.max_ctas / per < units_est) ? d.max_ctas / per : units_est;
        // (the warps address C themselves, so unlike the TMA-stored boxes this path also serves batched launches)
        const bool batch_ok = batch == 1 || (g.c_batch_stride * elem_size(d.c_type)) % 16 == 0;
        const bool can = c_tma_storable(d, g.c) && batch_ok && g.n_extra_c == 0 && ((d.n * elem_size(d.c_type)) % 16) == 0 &&
                         !(o.gemm_staged_store == 0 || o.gemm_staged_store == 1);
        if (can && (o.gemm_staged_store == 2 || short_k_epilogue(g, tiles_total <= units_cap))) { p.lsu_stage = 1; p.tma_store = 0; }
        p.c_in = (p.lsu_stage && d.beta != 0.0f && (o.gemm_c_in >= 0 ? o.gemm_c_in : 1)) ? 1 : 0;
        p.epi_warps = (p.lsu_stage && o.gemm_epi_warps != 4) ? 2 * kEpiWarps : kEpiWarps;
    }
    for (int r = 0; r < kMaxReplicas - 1; ++r) p.peer_c[r] = r < g.n_extra_c ? g.extra_c[r] : nullptr;
    // Forwarding CTAs: with three or more replicas to feed, the bytes leaving for other GPUs are a large share of
    // the launch and are better sent from SMs of their own (see copy_tiles).  With one or two the epilogue's own
    // stores cost less than the SMs would.
    p.copy_ctas = 0;
    p.tile_flags = nullptr;
    {
        const Options& o = options();
        const bool vec_rows = ((d.n * elem_size(d.c_type)) % 16) == 0;     // the forwarding stores are 16 bytes wide
        int want = o.gemm_copy_ctas >= 0 ? o.gemm_copy_ctas : (g.n_extra_c >= 6 ? 32 : g.n_extra_c >= 3 ? 18 : 0);
        want -= want % 2;
        if (g.n_extra_c > 0 && want > 0 && vec_rows && g.tile_flags && tiles_total <= g.tile_flags_capacity && want + 2 <= g.num_sms) {
            p.copy_ctas = want;
            p.tile_flags = g.tile_flags;
            cudaError_t fe = cudaMemsetAsync(p.tile_flags, 0, (size_t)tiles_total * sizeof(int), g.stream);
            if (fe != cudaSuccess) { *err = cudaGetErrorString(fe); return ACCB_ERR_CUDA; }
        }
    }
    if (p.pace_pct > 0) {
        static std::atomic<unsigned> next_slot{0};
        p.pace = g.status + kStatusWords + (next_slot.fetch_add(1) % kPaceSlots);
        cudaError_t pe = cudaMemsetAsync(p.pace, 0, sizeof(int), g.stream);
        if (pe != cudaSuccess) { *err = cudaGetErrorString(pe); return ACCB_ERR_CUDA; }
    }
    CReplicaMaps cm;
    memset(&cm, 0, sizeof cm);
    if (g.n_extra_c < 0 || g.n_extra_c > kMaxReplicas - 1) { *err = "tcgen05 GEMM: at most 7 extra C replicas"; return ACCB_ERR_ARG; }
    if (g.n_extra_c > 0 && !p.tma_store) { *err = "tcgen05 GEMM: C replicas need a row-major C with a 16-byte aligned pitch and base"; return ACCB_ERR_ARG; }
    if (p.tma_store) {
        bool ok = make_c_map(&cm.m[0], g.c, d.c_type, d.m, d.n, d.c_stride[0]);
        for (int r = 0; r < g.n_extra_c && ok; ++r) {
            if (!g.extra_c[r] || (reinterpret_cast<uintptr_t>(g.extra_c[r]) & 15)) { *err = "tcgen05 GEMM: C replica pointers must be non-null and 16-byte aligned"; return ACCB_ERR_ARG; }
            ok = make_c_map(&cm.m[1 + r], g.extra_c[r], d.c_type, d.m, d.n, d.c_stride[0]);
        }
        if (!ok) { *err = "tcgen05 GEMM: cuTensorMapEncodeTiled failed for C"; return ACCB_ERR_CUDA; }
    }
    p.status = g.status;
    if (tiles_total > 0x3fffffff) { *err = "tcgen05 GEMM: too many tiles"; return ACCB_ERR_ARG; }

#define ACCB_UMMA_LAUNCH(KIND, TC)                                                                          \
    (two_sm ? (bn == 256 ? launch_variant<KIND, TC, true, 256>(g, ma, mb, cm, p, err)                       \
                         : launch_variant<KIND, TC, true, 128>(g, ma, mb, cm, p, err))                      \
            : (bn == 256 ? launch_variant<KIND, TC, false, 256>(g, ma, mb, cm, p, err)                      \
                         : launch_variant<KIND, TC, false, 128>(g, ma, mb, cm, p, err)))

    if (d.a_type == ACCB_F16 || d.a_type == ACCB_BF16) {
        if (d.c_type == ACCB_F32) return ACCB_UMMA_LAUNCH(KIND_F16, float);
        if (d.c_type == ACCB_F16) return ACCB_UMMA_LAUNCH(KIND_F16, __half);
        return ACCB_UMMA_LAUNCH(KIND_F16, __nv_bfloat16);
    }
    if (d.a_type == ACCB_F32) return ACCB_UMMA_LAUNCH(KIND_TF32, float);
    return ACCB_UMMA_LAUNCH(KIND_I8, int32_t);
#undef ACCB_UMMA_LAUNCH
}

}  // namespace accb
