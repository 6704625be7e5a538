// Per-token layer chain on the 5th-generation tensor cores (bf16 mode).
//
// One CTA owns 128 token rows and walks the same chain as the fp32 kernel
// (out-proj + LN2 + MLP + LN3 [+ final LN + mixture head] [+ next layer's
// feature fold + LN1 + QKV + KV scatter]).  Every GEMM is tcgen05.mma with the
// accumulator in tensor memory:
//   * activations are split into a bf16 hi and lo part (x = hi + lo, 16 mantissa
//     bits) so that the products keep near-fp32 accuracy: rounding activations to
//     plain bf16 moves the log density by 1.5e-2, far outside the 2e-3 bar;
//   * the D-wide activation operand lives in TMEM (written by the epilogue threads
//     with tcgen05.st, read as the A operand), the 64-wide hidden tile of the MLP
//     goes through shared memory (swizzled K-major, written by the epilogue);
//   * weights are bf16 hi(/lo) tiles pre-swizzled on the host into the exact
//     shared-memory image, streamed by two producer warps with plain bulk copies
//     through two 3-slot rings (full / empty mbarriers).
// Warp 0: weight producer A.  Warp 1: MMA issuer A, owns the 512 TMEM columns.
// Warps 2-17: 512 epilogue threads, four per row (each owns a quarter of the
// columns); LayerNorm statistics are exchanged through shared memory.
// Warp 18: MMA issuer B (second GEMM of the MLP).  Warp 19: its weight producer.
// With few row tiles in flight a cluster of two CTAs shares one tile: see the
// kernel body.  All mbarrier waits are bounded; on expiry the CTA flags an
// abort, stops producing results, drains and frees TMEM.
#include <cstdlib>

#include "dense.cuh"
#include "kv_scatter.cuh"

namespace artab {

namespace {

constexpr int BM = 128;          // token rows per CTA
constexpr int HT = 128;          // hidden units per MLP tile
constexpr int NSLOT = 3;         // depth of each of the two weight rings
constexpr int NWG = 4;           // epilogue threads per row (column groups)
constexpr int kEpi = 128 * NWG;  // epilogue threads
constexpr int kThreads = 64 + kEpi + 64;  // + second MMA issuer warp and its weight producer warp
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccA = 0;    // wide accumulator (<= 192 columns)
constexpr uint32_t kAxHi = 192;  // activation operand, hi part (<= 96 packed columns)
constexpr uint32_t kAxLo = 288;  // activation operand, lo part
constexpr uint32_t kAccH = 384;  // hidden-tile accumulator, 128 columns
constexpr long long kWaitCycles = 2000000000LL;
constexpr int kPairMaxCtas = 148;  // CTA pairs only while all of them fit on the GPU at once

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(b, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try(b, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// mbarrier wait that also acquires what another CTA of the cluster released before its remote arrive
__device__ __forceinline__ bool mbar_try_cluster(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_cluster(b, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}
// ---- thread-block cluster (a pair of CTAs shares one 128-row tile) ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// split form: arrive right after the own barriers are initialised, wait only before the first access to
// the peer's shared memory (by then the peer has arrived long ago, so the wait costs nothing)
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared-memory address of the same object in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t raddr) {  // releases this thread's earlier stores
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(raddr) : "memory");
}

constexpr uint64_t kLayoutSw128 = 2;
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {  // K-major, 128-byte swizzle, 8-row groups 1 KiB apart
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= kLayoutSw128 << 61;
  return d;
}
// The issuing thread shares its scheduler with four busy epilogue warps, so every instruction it
// spends between two MMAs costs about five cycles: descriptors are built once per slab and
// stepped with a single add (the start-address field counts 16-byte units).
__device__ __forceinline__ uint64_t desc_step(uint64_t d, int bytes) { return d + (uint64_t)(bytes >> 4); }
__device__ __forceinline__ uint32_t make_idesc(int N) {  // M 128, fp32 accumulate, bf16 x bf16, K-major both
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_commit_addr(uint32_t cluster_addr) {  // a barrier of any CTA of the cluster
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// x -> (hi, lo) bf16 with hi + lo = x to 16 mantissa bits, for two neighbouring columns at once
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(a, b);
  lo = pack_bf16(a - __uint_as_float(hi << 16), b - __uint_as_float(hi & 0xffff0000u));
}

// Two fp32 operations per issued instruction (fma / add / mul .f32x2 on a register pair): the epilogue
// phases are bound by instruction issue on one SM, not by the fp32 pipe.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }

// GELU with erf(z) = 1 - 2^q(z) for z >= 0, q a degree-8 polynomial fitted to log2(erfc) on [0, 4]
// (|erf error| < 4e-6, below the 2^-17 of the hi + lo operand split): one MUFU op per element.
__device__ __forceinline__ float gelu_fast(float x) {
  const float z = fminf(fabsf(x) * 0.70710678118654752f, 6.0f);
  float q = fmaf(-1.2271906e-06f, z, -2.4917551e-06f);
  q = fmaf(q, z, 0.00038366718f);
  q = fmaf(q, z, -0.0049292254f);
  q = fmaf(q, z, 0.03347154f);
  q = fmaf(q, z, -0.15211754f);
  q = fmaf(q, z, -0.9171586f);
  q = fmaf(q, z, -1.6280657f);
  q *= z;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(q));
  const float h = 0.5f * x;
  return fmaf(copysignf(1.0f - e, x), h, h);  // 0.5 x (1 + erf)
}


// Optional in-kernel timeline (diagnostic builds only, -DARTAB_TIMELINE; read by
// `microbench.py timeline`): the first epilogue thread of every CTA stamps clock64() at the phase
// boundaries of the launch; slot = launch counter mod 32.  Marks: 0 roles split, 1 constants staged,
// 2 predecessor complete, 3 attention rows published, 4 Wo accumulator ready, 25 LayerNorm 2 done,
// 5 x2 published, 6 MLP starts, 7.. hidden tile done, 13 second GEMM complete, 10 / 11 / 12 / 19
// exchange (enter, peer ready, stores issued, data arrived), 14 exchange done, 15 LayerNorm 3 done,
// 16 x3 published, 17 fold accumulator ready, 18 x1 published, 27 issuer sees x1, 20 / 22 projection
// accumulators ready, 21 / 23 staged projections stored, 24 head accumulator ready, 26 epilogue done;
// 28 clock at kernel entry; 29 / 30 / 31 global timer (ns) at entry, predecessor complete, end.
#ifdef ARTAB_TIMELINE
__device__ long long g_tl[32][32][32];   // [launch slot][cta][mark]
#define TL(id) do { if (tl_on) g_tl[a.tl_slot & 31][blockIdx.x & 31][id] = clock64(); } while (0)
__device__ __forceinline__ long long gtimer() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define TLG(id) do { if (tl_on) g_tl[a.tl_slot & 31][blockIdx.x & 31][id] = gtimer(); } while (0)
#define TLS(event) do { if (tl_on) ARTAB_STAMP(1, event); } while (0)
#else
#define TL(id) do { } while (0)
#define TLG(id) do { } while (0)
#define TLS(event) do { } while (0)
#endif

// The same for two neighbouring columns at once, on packed pairs (same operations, same rounding as
// gelu_fast; sign(x) * (1 - e) * x / 2 is written (1 - e) * |x| / 2, which is the same product).
__device__ __forceinline__ float2 gelu_fast2(float2 x) {
  const float2 ax = make_float2(fabsf(x.x), fabsf(x.y));
  float2 z = mul2(ax, splat2(0.70710678118654752f));
  z.x = fminf(z.x, 6.0f);
  z.y = fminf(z.y, 6.0f);
  float2 q = fma2(splat2(-1.2271906e-06f), z, splat2(-2.4917551e-06f));
  q = fma2(q, z, splat2(0.00038366718f));
  q = fma2(q, z, splat2(-0.0049292254f));
  q = fma2(q, z, splat2(0.03347154f));
  q = fma2(q, z, splat2(-0.15211754f));
  q = fma2(q, z, splat2(-0.9171586f));
  q = fma2(q, z, splat2(-1.6280657f));
  q = mul2(q, z);
  float2 e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(q.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(q.y));
  const float2 t = fma2(e, splat2(-1.0f), splat2(1.0f));   // 1 - e, exact like the subtraction
  const float2 h = mul2(x, splat2(0.5f));
  return fma2(t, mul2(ax, splat2(0.5f)), h);               // 0.5 x (1 + erf)
}

struct __align__(1024) Smem {
  uint8_t ring[2][NSLOT][192 * 128];  // two weight rings (first / second MLP GEMM), slabs <= d_model * 128 bytes
  uint8_t ah[2][2][BM * 128];         // hidden tile operand [hi, lo][k-chunk][128 rows x 64 bf16], swizzled
  float xs[2 * NWG][BM];              // LayerNorm partial statistics (mean, M2) exchanged between the column groups
  float bias_h[1024];                 // hidden bias of the current MLP (b1 / head.0 bias), d_ff <= 1024
  float vec[8][192];                  // ln2 g,b | b2 | ln3 g,b | (ln1 | final) g,b | spare
  __nv_bfloat16* rowdst[BM];          // private-buffer K slot of each row's token (null: not cached)
  uint64_t w_full[2][NSLOT], w_empty[2][NSLOT];
  uint64_t ep_done, acc_full, h_full, acch_free, ah_ready, ah_free;
  uint64_t x_full;   // CTA pair: the peer's partial sums have arrived (MLP: in this CTA's landing zone; head: in the global scratch)
  uint64_t x_ready;  // CTA pair: the peer's landing zone (its second weight ring + hidden-operand buffers) is idle
  uint64_t x_done;   // CTA pair: every epilogue thread has read the landing zone: the second weight ring may be refilled
  uint32_t tmem_base;
  int abort_flag;
};

static_assert(sizeof(Smem) + 1024 <= 227 * 1024, "shared-memory plan exceeds what one CTA may request");

__device__ __forceinline__ bool direct_mode(int mode) { return mode == KV_PREFILL; }

struct Ctx {
  Smem* sm;
  volatile int* abort_flag;
  uint32_t tmem;
};

// ------------------------------------------------------------------ producer
struct Producer {
  Smem* sm;
  int ring;   // which weight ring this thread feeds
  int issued;
  bool ok;
  __device__ void slab(const uint8_t* src, uint32_t bytes) {
    if (!ok) return;
    const int buf = issued % NSLOT;
    if (issued >= NSLOT && !mbar_wait(&sm->w_empty[ring][buf], ((issued / NSLOT) + 1) & 1, &sm->abort_flag)) {
      ok = false;
      return;
    }
    uint64_t* bar = &sm->w_full[ring][buf];
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(sm->ring[ring][buf])), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
    ++issued;
  }
  // all slabs of a matrix consumed in order ("full" layout: one k-chunk group after the other)
  __device__ void matrix(const void* w, int groups, bool has_lo, uint32_t slab_bytes) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(w);
    const int n = groups * (has_lo ? 2 : 1);
    for (int i = 0; i < n; ++i) slab(p + (size_t)i * slab_bytes, slab_bytes);
  }
  // first GEMM of an MLP: per 128-wide hidden tile nkc slabs of 16 KB per part
  // (hidden tiles first, first + step, ... < nt: a CTA pair shares the tiles of one MLP)
  __device__ void mlp_first(const void* w1, bool lo1, int nkc, int nt, int first, int step) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(w1);
    const int per = nkc * (lo1 ? 2 : 1);  // tile-major: hi k-chunks then lo k-chunks of every tile
    for (int j = first; j < nt; j += step)
      for (int i = 0; i < per; ++i) slab(p + (size_t)(j * per + i) * (HT * 128), HT * 128);
  }
  // second GEMM of an MLP: per hidden tile two k-chunk slabs per part
  __device__ void mlp_second(const void* w2, bool lo2, uint32_t bytes2, int nt, int first, int step) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(w2);
    const int per = 2 * (lo2 ? 2 : 1);
    for (int j = first; j < nt; j += step)
      for (int i = 0; i < per; ++i) slab(p + (size_t)(j * per + i) * bytes2, bytes2);
  }
  // k-chunk groups [g0, g1) of a "full" matrix stack
  __device__ void matrix_range(const void* w, int g0, int g1, bool has_lo, uint32_t slab_bytes) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(w);
    const int per = has_lo ? 2 : 1;
    for (int i = g0 * per; i < g1 * per; ++i) slab(p + (size_t)i * slab_bytes, slab_bytes);
  }
};

// ---------------------------------------------------------------- MMA issuer
struct Issuer {
  Smem* sm;
  uint32_t tmem;
  int ring;         // which weight ring this thread drains
  int consumed;     // ring slabs consumed
  int ep_phase;     // completed waits on ep_done
  int ah_count;     // completed waits on ah_ready
  int hfree_count;  // completed waits on acch_free
  bool ok;

  __device__ uint32_t slab_wait() {
    const int buf = consumed % NSLOT;
    ok = ok && mbar_wait(&sm->w_full[ring][buf], (consumed / NSLOT) & 1, &sm->abort_flag);
    tc_fence_after();
    return smem_u32(sm->ring[ring][buf]);
  }
  __device__ void slab_release() {
    umma_commit(&sm->w_empty[ring][consumed % NSLOT]);
    ++consumed;
  }
  __device__ void wait_epilogue() {
    ok = ok && mbar_wait(&sm->ep_done, ep_phase & 1, &sm->abort_flag);
    ++ep_phase;
    tc_fence_after();
  }
  // ACC[acc_col] = A_x . W^T with W streamed as `nkc` slabs of [n_out rows][64 k].
  // One out-of-line copy serves every call site (see gemm_full_ts_shared below).
  __device__ void gemm_full_ts(uint32_t acc_col, int n_out, int nkc, bool has_lo);
  // ACC_H (128 columns) = A_x . W_tile^T; the tile arrives as nkc slabs of [128 rows][64 k] per part,
  // ordered hi part (all k-chunks) then lo part
  __device__ void gemm_tile_ts(int nkc, bool has_lo) {
    const uint32_t idesc = make_idesc(HT);
    const uint32_t acc = tmem + kAccH;
    uint32_t ahi = tmem + kAxHi, alo = tmem + kAxLo;
    for (int kc = 0; kc < nkc; ++kc, ahi += 32, alo += 32) {
      const uint64_t bd = make_desc(slab_wait());
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_ts(acc, ahi + ks * 8, desc_step(bd, 32 * ks), idesc, (kc | ks) != 0);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_ts(acc, alo + ks * 8, desc_step(bd, 32 * ks), idesc, 1);
      slab_release();
    }
    if (has_lo) {
      ahi = tmem + kAxHi;
      for (int kc = 0; kc < nkc; ++kc, ahi += 32) {
        const uint64_t ld = make_desc(slab_wait());
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_ts(acc, ahi + ks * 8, desc_step(ld, 32 * ks), idesc, 1);
        slab_release();
      }
    }
  }
  // ACC_A (+)= A_h . W_chunks^T for the two 64-wide k-chunks of one hidden tile (A from shared memory)
  __device__ void gemm_chunks_ss(int n_out, bool has_lo, bool accumulate) {
    const uint32_t idesc = make_idesc(n_out);
    const uint32_t acc = tmem + kAccA;
    for (int kc = 0; kc < 2; ++kc) {
      const uint64_t a_hi = make_desc(smem_u32(sm->ah[0][kc])), a_lo = make_desc(smem_u32(sm->ah[1][kc]));
      const uint64_t bd = make_desc(slab_wait());
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_ss(acc, desc_step(a_hi, 32 * ks), desc_step(bd, 32 * ks), idesc, accumulate || (kc | ks) != 0);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_ss(acc, desc_step(a_lo, 32 * ks), desc_step(bd, 32 * ks), idesc, 1);
      slab_release();
      if (has_lo) {
        const uint64_t ld = make_desc(slab_wait());
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_ss(acc, desc_step(a_hi, 32 * ks), desc_step(ld, 32 * ks), idesc, 1);
        slab_release();
      }
    }
  }
  // First MLP GEMM (issuer A): hidden tile j = A_x . W1_j^T into ACC_H.  The epilogue frees ACC_H
  // as soon as it has pulled a tile into registers, so tile j+1 is computed while tile j is still
  // being activated.
  __device__ void mlp_first(int nkc, bool lo1, int nt) {
    for (int j = 0; j < nt; ++j) {
      if (j >= 1) wait_hidden_free();
      gemm_tile_ts(nkc, lo1);
      umma_commit(&sm->h_full);
    }
    wait_hidden_free();  // keeps the phase count exact for a second MLP in the same launch
  }
  // Second MLP GEMM (issuer B, its own thread: MMAs from two threads overlap in the tensor pipe):
  // ACC_A (+)= act(hidden tile j) . W2_j^T as soon as the epilogue has published tile j.
  __device__ void mlp_second(bool lo2, int nt, int n_out) {
    for (int j = 0; j < nt; ++j) {
      ok = ok && mbar_wait(&sm->ah_ready, ah_count & 1, &sm->abort_flag);
      ++ah_count;
      tc_fence_after();
      gemm_chunks_ss(n_out, lo2, j > 0);
      umma_commit(&sm->ah_free);
    }
    umma_commit(&sm->acc_full);
  }
  __device__ void wait_hidden_free() {
    ok = ok && mbar_wait(&sm->acch_free, hfree_count & 1, &sm->abort_flag);
    ++hfree_count;
    tc_fence_after();
  }
};

// The issuing thread walks this code alone: every inlined copy of it would be a stretch of cold
// instructions (thousands of cycles of fetch stalls per GEMM were measured with one copy per call
// site).  So there is ONE copy, entered with everything in registers; it returns the new ring count,
// or -1 - count when a wait gave up.
__device__ __noinline__ int gemm_full_ts_shared(Smem* sm, uint32_t tmem, int ring, int consumed, uint32_t acc_col,
                                                int n_out, int nkc, int has_lo) {
  const uint32_t idesc = make_idesc(n_out);
  const uint32_t acc = tmem + acc_col;
  uint32_t ahi = tmem + kAxHi, alo = tmem + kAxLo;
  bool ok = true;
  for (int kc = 0; kc < nkc; ++kc, ahi += 32, alo += 32) {
    int buf = consumed % NSLOT;
    ok = ok && mbar_wait(&sm->w_full[ring][buf], (consumed / NSLOT) & 1, &sm->abort_flag);
    tc_fence_after();
    const uint64_t bd = make_desc(smem_u32(sm->ring[ring][buf]));
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) umma_ts(acc, ahi + ks * 8, desc_step(bd, 32 * ks), idesc, (kc | ks) != 0);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) umma_ts(acc, alo + ks * 8, desc_step(bd, 32 * ks), idesc, 1);
    umma_commit(&sm->w_empty[ring][buf]);
    ++consumed;
    if (has_lo) {
      buf = consumed % NSLOT;
      ok = ok && mbar_wait(&sm->w_full[ring][buf], (consumed / NSLOT) & 1, &sm->abort_flag);
      tc_fence_after();
      const uint64_t ld = make_desc(smem_u32(sm->ring[ring][buf]));
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_ts(acc, ahi + ks * 8, desc_step(ld, 32 * ks), idesc, 1);
      umma_commit(&sm->w_empty[ring][buf]);
      ++consumed;
    }
  }
  return ok ? consumed : -1 - consumed;
}
__device__ __forceinline__ void Issuer::gemm_full_ts(uint32_t acc_col, int n_out, int nkc, bool has_lo) {
  const int r = gemm_full_ts_shared(sm, tmem, ring, consumed, acc_col, n_out, nkc, has_lo ? 1 : 0);
  if (r < 0) {
    ok = false;
    consumed = -1 - r;
  } else {
    consumed = r;
  }
}

// ------------------------------------------------------------------ epilogue
template <int D>
struct Epilogue {
  static constexpr int PART = D / NWG;     // columns owned by one thread
  static constexpr int NCH = PART / 16;    // 16-column chunks
  static constexpr int HPART = HT / NWG;   // hidden-tile columns owned by one thread (16)
  Smem* sm;
#ifdef ARTAB_TIMELINE
  int tl_slot;
#endif
  uint32_t t_row;                          // TMEM address of this thread's lane
  int row, wg, col0;
  int acc_phase, xs_phase;
  int h_count, free_count;
  bool ok;

  __device__ void sync_groups() { asm volatile("bar.sync 3, %0;" ::"n"(kEpi) : "memory"); }
  // only the four warps that own this row quadrant (one per column group) meet
  __device__ void quadrant_sync() { asm volatile("bar.sync %0, 128;" ::"r"(4 + (row >> 5)) : "memory"); }

  __device__ void wait_acc() {
    ok = mbar_wait(&sm->acc_full, acc_phase & 1, &sm->abort_flag) && ok;
    ++acc_phase;
    tc_fence_after();
  }
  // v[i] += ACC_A[col0 + i]   (16 columns at a time: keeps the live register set small)
  __device__ void add_acc(float* v) {
    uint32_t r[16];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      tmem_ld16(t_row + kAccA + col0 + 16 * c, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) v[16 * c + i] += __uint_as_float(r[i]);
    }
  }
  // A_x <- split(v) for this thread's columns, then tell the MMA warp
  __device__ void publish_ax(const float* v) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) split2(v[16 * c + 2 * i], v[16 * c + 2 * i + 1], hi[i], lo[i]);
      tmem_st8(t_row + kAxHi + (col0 >> 1) + 8 * c, hi);
      tmem_st8(t_row + kAxLo + (col0 >> 1) + 8 * c, lo);
    }
    done();
  }
  // v <- hi + lo of this thread's columns of the activation operand: what publish_ax stored, i.e. the
  // published values to 2^-18 relative.  The MLP's residual x2 is read back this way after the MLP
  // (the operand stays in tensor memory until the next publish) instead of waiting in a workspace.
  __device__ void load_ax(float* v) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      uint32_t hi[8], lo[8];
      tmem_ld8(t_row + kAxHi + (col0 >> 1) + 8 * c, hi);
      tmem_ld8(t_row + kAxLo + (col0 >> 1) + 8 * c, lo);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[16 * c + 2 * i] = __uint_as_float(hi[i] << 16) + __uint_as_float(lo[i] << 16);
        v[16 * c + 2 * i + 1] = __uint_as_float(hi[i] & 0xffff0000u) + __uint_as_float(lo[i] & 0xffff0000u);
      }
    }
  }
  __device__ void done() {
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(&sm->ep_done);
  }
  // LayerNorm over the full row (NWG threads, one per column group).  Every thread takes the mean and
  // the sum of squared deviations of its own columns (two local passes, no cancellation); the groups
  // are then combined with the pairwise-variance update after ONE exchange through shared memory, in a
  // fixed order (deterministic).  Pairs of columns go through the packed fp32 instructions, gamma /
  // beta come as 16-byte shared-memory loads.
  __device__ void layer_norm(float* v, const float* gamma, const float* beta) {
    float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < PART; i += 2) s2 = add2(s2, make_float2(v[i], v[i + 1]));
    const float lmean = (s2.x + s2.y) * (1.0f / (float)PART);
    const float2 nl = splat2(-lmean);
    float2 ss2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < PART; i += 2) {
      const float2 d = add2(make_float2(v[i], v[i + 1]), nl);
      ss2 = fma2(d, d, ss2);
    }
    // The exchange buffer is single: two LayerNorms of one launch are always separated by an
    // accumulator wait that every epilogue thread passes (so nobody still reads the old statistics),
    // except the final LayerNorm, which follows the last layer's directly: quadrant_sync() before it.
    sm->xs[wg][row] = lmean;
    sm->xs[NWG + wg][row] = ss2.x + ss2.y;
    quadrant_sync();
    float msum = 0.f, m2 = 0.f, gm[NWG];
#pragma unroll
    for (int g = 0; g < NWG; ++g) {
      gm[g] = sm->xs[g][row];
      msum += gm[g];
      m2 += sm->xs[NWG + g][row];
    }
    const float mean = msum * (1.0f / (float)NWG);
    float dev = 0.f;
#pragma unroll
    for (int g = 0; g < NWG; ++g) dev = fmaf(gm[g] - mean, gm[g] - mean, dev);
    const float var = fmaf((float)PART, dev, m2) * (1.0f / (float)D);
    const float2 rstd = splat2(rsqrtf(var + 1e-5f));
    const float2 nm = splat2(-mean);
#pragma unroll
    for (int i = 0; i < PART; i += 4) {
      const float4 g = *reinterpret_cast<const float4*>(gamma + col0 + i);
      const float4 b = *reinterpret_cast<const float4*>(beta + col0 + i);
      const float2 y0 = fma2(mul2(add2(make_float2(v[i], v[i + 1]), nm), rstd), make_float2(g.x, g.y), make_float2(b.x, b.y));
      const float2 y1 = fma2(mul2(add2(make_float2(v[i + 2], v[i + 3]), nm), rstd), make_float2(g.z, g.w), make_float2(b.z, b.w));
      v[i] = y0.x; v[i + 1] = y0.y; v[i + 2] = y1.x; v[i + 3] = y1.y;
    }
  }
  // hidden tile j: act(ACC_H + bias) -> split -> swizzled shared-memory operand
  // (jl counts this CTA's tiles, j is the tile's index in the MLP)
  __device__ void hidden_tile(int jl, int j, const float* bias) {
    ok = mbar_wait(&sm->h_full, h_count & 1, &sm->abort_flag) && ok;
    ++h_count;
    tc_fence_after();
    uint32_t r[2][16];
#pragma unroll
    for (int c = 0; c < 2; ++c) tmem_ld16(t_row + kAccH + HPART * wg + 16 * c, r[c]);
    tmem_wait_ld();
    tc_fence_before();
    mbar_arrive(&sm->acch_free);  // the accumulator is in registers: the next tile's GEMM may overwrite it
    uint32_t hi[16], lo[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float4 bb = *reinterpret_cast<const float4*>(bias + j * HT + HPART * wg + 2 * i);
      const float2 a0 = make_float2(__uint_as_float(r[i >> 3][(2 * i) & 15]), __uint_as_float(r[i >> 3][(2 * i + 1) & 15]));
      const float2 a1 = make_float2(__uint_as_float(r[i >> 3][(2 * i + 2) & 15]), __uint_as_float(r[i >> 3][(2 * i + 3) & 15]));
      const float2 g0 = gelu_fast2(add2(a0, make_float2(bb.x, bb.y)));
      const float2 g1 = gelu_fast2(add2(a1, make_float2(bb.z, bb.w)));
      split2(g0.x, g0.y, hi[i], lo[i]);
      split2(g1.x, g1.y, hi[i + 1], lo[i + 1]);
    }
    if (jl >= 1) {  // the previous tile's second GEMM must have finished reading the operand buffer
      ok = mbar_wait(&sm->ah_free, free_count & 1, &sm->abort_flag) && ok;
      ++free_count;
    }

    // this thread's 32 hidden columns sit in k-chunk wg / 2, 16-byte chunks 4 * (wg % 2) .. + 3 of the
    // 128-byte row; chunk c of row r lives at chunk position c ^ (r % 8)
    uint8_t* base_hi = sm->ah[0][wg >> 1] + row * 128;
    uint8_t* base_lo = sm->ah[1][wg >> 1] + row * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int pos = ((4 * (wg & 1) + c) ^ (row & 7)) * 16;
      *reinterpret_cast<uint4*>(base_hi + pos) = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
      *reinterpret_cast<uint4*>(base_lo + pos) = make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA's reads
    tc_fence_before();
    mbar_arrive(&sm->ah_ready);
  }
  // After an MLP: consume the ah_free completion of its last tile, which no hidden_tile waited for,
  // so that the parity bookkeeping is exact when a second MLP runs in the same launch.
  __device__ void drain_free() {
    ok = mbar_wait(&sm->ah_free, free_count & 1, &sm->abort_flag) && ok;
    ++free_count;
  }
  // CTA pair: v[i] += (own MLP partial + the peer's).  Each CTA holds the second GEMM's sum over its
  // half of the hidden tiles in ACC_A.  The partials cross through distributed shared memory: once a
  // CTA's own second GEMM is complete, its second weight ring and hidden-operand buffers are idle
  // and serve as the landing zone (96 KB, float4 column groups outermost, the 128 rows innermost, so
  // a warp's stores and loads are contiguous 512-byte spans).  Hand-shake: tell the peer that this
  // CTA's zone is free, wait for the peer's word, store the own partial into the PEER's zone,
  // release-arrive on the peer's barrier, acquire-wait on the own one, read the own zone.
  // a + b == b + a exactly, so both CTAs end up with the same bits.  Called after wait_acc().
  // Remote arrivals are single transactions on the cluster network, so they are kept few: "zone free"
  // is ONE arrival, made by the tensor core itself (the second issuer commits its last MMAs of the MLP
  // onto the PEER's barrier), "partial delivered" is one arrival per warp (__syncwarp orders the
  // warp's stores before lane 0's release).  The exchange is split in two so that the caller can put
  // independent work (reading the residual back, adding the bias) between sending and receiving.
#ifdef ARTAB_TIMELINE
#define XTL(id) do { if (threadIdx.x == 64) g_tl[tl_slot & 31][blockIdx.x & 31][id] = clock64(); } while (0)
#else
#define XTL(id) do { } while (0)
#endif
  __device__ void send_partial(uint32_t peer) {
    XTL(10);
    ok = mbar_wait_cluster(&sm->x_ready, 0, &sm->abort_flag) && ok;   // the peer's zone is idle
    XTL(11);
    const uint32_t zone_peer = map_to_rank(smem_u32(&sm->ring[1][0][0]), peer);
    uint32_t r[16];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      tmem_ld16(t_row + kAccA + col0 + 16 * c, r);
      tmem_wait_ld();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t dst = zone_peer + (uint32_t)((((col0 >> 2) + 4 * c + q) * BM + row) * 16);
        asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(r[4 * q]), "r"(r[4 * q + 1]),
                     "r"(r[4 * q + 2]), "r"(r[4 * q + 3])
                     : "memory");
      }
    }
    XTL(12);
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive_remote(map_to_rank(smem_u32(&sm->x_full), peer));  // releases the warp's stores
  }
  __device__ void receive_add(float* v) {
    ok = mbar_wait_cluster(&sm->x_full, 0, &sm->abort_flag) && ok;
    XTL(19);
    const float4* zone = reinterpret_cast<const float4*>(&sm->ring[1][0][0]);
    uint32_t r[16];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float4 t[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) t[q] = zone[((col0 >> 2) + 4 * c + q) * BM + row];
      tmem_ld16(t_row + kAccA + col0 + 16 * c, r);
      tmem_wait_ld();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        v[16 * c + 4 * q] += __uint_as_float(r[4 * q]) + t[q].x;
        v[16 * c + 4 * q + 1] += __uint_as_float(r[4 * q + 1]) + t[q].y;
        v[16 * c + 4 * q + 2] += __uint_as_float(r[4 * q + 2]) + t[q].z;
        v[16 * c + 4 * q + 3] += __uint_as_float(r[4 * q + 3]) + t[q].w;
      }
    }
    mbar_arrive(&sm->x_done);  // the values above are in registers: the zone may be overwritten
  }
};

// Mixture head for one row from raw[3K] (one thread): sample or log-pdf.
__device__ __forceinline__ void head_row_thread(const DenseArgs& a, const float* raw, long row) {
  const int K = a.n_comp;
  const long b = row / a.head_tps;
  const int j = (int)(row - b * a.head_tps);
  if (j < a.head_first) return;
  const long oidx = b * a.out_stride + a.out_col + (j - a.head_first);
  float mean[8], stdv[8], lw[8];
  float mx = -INFINITY;
  for (int k = 0; k < K; ++k) {
    mean[k] = raw[3 * k] + __ldg(a.mean_bias + k);
    const float sr = raw[3 * k + 1] + __ldg(a.std_bias + k);
    const float sp = sr > 20.f ? sr : log1pf(expf(sr));
    stdv[k] = fminf(sp, 2.0f) + 1e-3f;
    lw[k] = raw[3 * k + 2] + __ldg(a.weight_bias + k);
    mx = fmaxf(mx, lw[k]);
  }
  float se = 0.f;
  for (int k = 0; k < K; ++k) se += expf(lw[k] - mx);
  const float lse = mx + logf(se);
  float y;
  if (a.head_mode == 1) {
    int best = 0;
    float bv = -1.f;
    for (int k = 0; k < K; ++k) {
      const float ratio = expf(lw[k] - lse) / __ldg(a.expo + b * K + k);
      if (ratio > bv) {
        bv = ratio;
        best = k;
      }
    }
    y = mean[best] + stdv[best] * __ldg(a.normal + b);
    a.y_out[oidx] = y;
    if (a.comp_out) a.comp_out[oidx] = best;
  } else {
    y = __ldg(a.y_in + oidx);
  }
  if (a.ld_out) {
    float lp[8], m2 = -INFINITY;
    for (int k = 0; k < K; ++k) {
      const float zz = (y - mean[k]) / stdv[k];
      lp[k] = -0.5f * (1.8378770664093453f + 2.0f * logf(stdv[k]) + zz * zz) + (lw[k] - lse);
      m2 = fmaxf(m2, lp[k]);
    }
    float s2 = 0.f;
    for (int k = 0; k < K; ++k) s2 += expf(lp[k] - m2);
    a.ld_out[oidx] = m2 + logf(s2);
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1) dense_tc_kernel(const DenseArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Smem* sm = reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ARTAB_TIMELINE
  if (threadIdx.x == 64) {
    g_tl[a.tl_slot & 31][blockIdx.x & 31][29] = gtimer();
    g_tl[a.tl_slot & 31][blockIdx.x & 31][28] = clock64();
    ARTAB_STAMP(1, 0);
  }
#endif
  constexpr int NKC = D / 64;
  constexpr uint32_t kSlab = D * 128;

  // The epilogue threads fetch the per-column constants (LayerNorm vectors, biases: model constants,
  // nothing the preceding kernel wrote) before anything else, into registers: the loads are in flight
  // while the barriers are set up and tensor memory is allocated, and are stored to shared memory
  // once the roles have split.  All loads are issued before the first store (read-only path: the
  // compiler may not assume that the shared-memory stores leave the global vectors alone, and would
  // otherwise wait for every load in turn).
  constexpr int kBiasPerThread = (1024 + kEpi - 1) / kEpi;
  float cv[7], cb[kBiasPerThread];
  {
    const int i = (int)threadIdx.x - 64;
    const bool epi = i >= 0 && i < kEpi;
    const bool col = epi && i < D;
#pragma unroll
    for (int k = 0; k < 7; ++k) cv[k] = 0.f;
    if (col && a.do_post) {
      cv[0] = __ldg(a.post_w.ln2_g + i);
      cv[1] = __ldg(a.post_w.ln2_b + i);
      cv[2] = __ldg(a.post_w.b2 + i);
      cv[3] = __ldg(a.post_w.ln3_g + i);
      cv[4] = __ldg(a.post_w.ln3_b + i);
    }
    if (col && a.do_final) {
      cv[5] = __ldg(a.lnf_g + i);
      cv[6] = __ldg(a.lnf_b + i);
    } else if (col && a.do_pre) {
      cv[5] = __ldg(a.pre_w.ln1_g + i);
      cv[6] = __ldg(a.pre_w.ln1_b + i);
    }
#pragma unroll
    for (int k = 0; k < kBiasPerThread; ++k)
      cb[k] = (epi && a.do_post && i + k * kEpi < a.Dff) ? __ldg(a.post_w.b1 + i + k * kEpi) : 0.f;
  }
  const int nt = a.Dff / HT;
  // A CTA pair (cluster of 2) may share one row tile: both walk the whole chain, but each takes
  // every other hidden tile of the layer's MLP (partial sums exchanged once) and a part of the
  // Q / K / V projections.  csize == 1: one CTA does everything.
  const uint32_t crank = cluster_rank(), csize = cluster_size();
  const long row0 = (long)(blockIdx.x / csize) * BM;
  const int t_begin = (csize == 2 && crank == 1) ? 2 : 0;   // projections (0 q, 1 k, 2 v) of this CTA
  const int t_end = (csize == 2 && crank == 0) ? 2 : 3;

  // barrier set-up spread over the first warp (one barrier per lane instead of one thread doing all)
  if (warp == 0) {
    if (lane < 2 * NSLOT) {
      mbar_init(&sm->w_full[lane / NSLOT][lane % NSLOT], 1);
      mbar_init(&sm->w_empty[lane / NSLOT][lane % NSLOT], 1);
    }
    switch (lane) {
      case 8: mbar_init(&sm->ep_done, kEpi); break;
      case 9: mbar_init(&sm->acc_full, 1); break;
      case 10: mbar_init(&sm->h_full, 1); break;
      case 11: mbar_init(&sm->acch_free, kEpi); break;
      case 12: mbar_init(&sm->ah_ready, kEpi); break;
      case 13: mbar_init(&sm->ah_free, 1); break;
      case 14: mbar_init(&sm->x_full, kEpi / 32); break;   // one remote arrival per epilogue warp
      case 15: mbar_init(&sm->x_ready, 1); break;          // one remote arrival per CTA
      case 16: mbar_init(&sm->x_done, kEpi); break;
      case 17: sm->abort_flag = 0; break;
      default: break;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The peer's barriers must exist before anyone arrives on them.  Every thread arrives here; the
  // epilogue threads wait just before the MLP exchange (the first remote access of a launch), all
  // other threads, and the epilogue threads of a launch without an exchange, at the end.
  if (csize > 1) cluster_arrive();
  bool cluster_waited = false;
  const uint32_t tmem = sm->tmem_base;

  const int lo_post = a.post_w.tc_lo, lo_pre = a.pre_w.tc_lo;
  const int n_mine = (nt - (int)crank + (int)csize - 1) / (int)csize;  // hidden tiles of the layer MLP done here
  // the head MLP is shared the same way (second exchange, its own scratch slots)
  const bool head_pair = csize > 1;
  const int h_first = head_pair ? (int)crank : 0, h_step = head_pair ? (int)csize : 1;
  const int h_mine = head_pair ? n_mine : nt;

  if (warp == 0) {
    // --------------------- weight producer A: everything but the second MLP GEMM ---------------------
    if (lane == 0) {
      Producer p{sm, 0, 0, true};
      if (a.do_post) {
        p.matrix(a.post_w.tc_wo, NKC, lo_post & 1, kSlab);
        p.mlp_first(a.post_w.tc_w1, lo_post & 2, NKC, nt, crank, csize);
      }
      if (a.do_head) {
        p.mlp_first(a.tc_wa, a.tc_head_lo & 1, NKC, nt, h_first, h_step);
      } else if (a.do_pre) {
        p.matrix(a.pre_w.tc_wf, NKC, lo_pre & 8, kSlab);
        // this CTA's projections alternate between the two rings, the first one in the SECOND ring:
        // that ring is idle once the MLP is over, so these weights are resident long before x1 is
        // published, while this ring is still busy with the folded feature-attention matrix
        for (int t = t_begin + 1; t < t_end; t += 2) p.matrix_range(a.pre_w.tc_wqkv, t * NKC, (t + 1) * NKC, lo_pre & 16, kSlab);
      }
    }
  } else if (warp == 19) {
    // --------------------- weight producer B: the second MLP GEMM's k-chunks ---------------------
    if (lane == 0) {
      Producer p{sm, 1, 0, true};
      if (a.do_post) p.mlp_second(a.post_w.tc_w2, lo_post & 4, kSlab, nt, crank, csize);
      // a pair uses this ring as the landing zone of the MLP exchange: nothing more goes into it
      // until every epilogue thread has read the zone
      if (a.do_post && csize > 1 && !mbar_wait(&sm->x_done, 0, &sm->abort_flag)) p.ok = false;
      if (a.do_head) {
        p.mlp_second(a.tc_wb, a.tc_head_lo & 2, 16 * 128, nt, h_first, h_step);
      } else if (a.do_pre) {
        for (int t = t_begin; t < t_end; t += 2) p.matrix_range(a.pre_w.tc_wqkv, t * NKC, (t + 1) * NKC, lo_pre & 16, kSlab);
      }
    }
  } else if (warp == 1) {
    // --------------------------------- MMA issuer A ---------------------------------
    if (lane == 0) {
      Issuer m{sm, tmem, 0, 0, 0, 0, 0, true};
      if (a.do_post) {
        m.wait_epilogue();                               // A_x = attention output
        m.gemm_full_ts(kAccA, D, NKC, lo_post & 1);
        umma_commit(&sm->acc_full);
        m.wait_epilogue();                               // A_x = x2 (and ACC_A drained)
        m.mlp_first(NKC, lo_post & 2, n_mine);
      }
      if (a.do_head) {
        m.wait_epilogue();                               // A_x = z
        m.mlp_first(NKC, a.tc_head_lo & 1, h_mine);
      } else if (a.do_pre) {
        m.wait_epilogue();                               // A_x = layer input
        m.gemm_full_ts(kAccA, D, NKC, lo_pre & 8);
        umma_commit(&sm->acc_full);
        m.wait_epilogue();                               // A_x = x1
#ifdef ARTAB_TIMELINE
        g_tl[a.tl_slot & 31][blockIdx.x & 31][27] = clock64();
#endif
        // second ring, continued where the second issuer left it (the MLP's second GEMM of this launch).
        // Both issuer states are used by name, never through a reference chosen at run time: that
        // would push them out of registers into the thread's stack, whose first touch is a cold miss.
        Issuer mb{sm, tmem, 1, a.do_post ? n_mine * 2 * ((lo_post & 4) ? 2 : 1) : 0, 0, 0, 0, true};
        for (int t = t_begin; t < t_end; ++t) {
          if (t > t_begin) m.wait_epilogue();            // previous projection drained from ACC_A
          if (((t - t_begin) & 1) == 0) {
            mb.ok = mb.ok && m.ok;
            mb.gemm_full_ts(kAccA, D, NKC, lo_pre & 16);
          } else {
            m.ok = m.ok && mb.ok;
            m.gemm_full_ts(kAccA, D, NKC, lo_pre & 16);
          }
          umma_commit(&sm->acc_full);
        }
      }
    }
  } else if (warp == 18) {
    // --------------------------------- MMA issuer B ---------------------------------
    if (csize > 1 && a.do_post) {  // whole warp: this thread will arrive on the peer's barrier
      cluster_wait();
      cluster_waited = true;
    }
    if (lane == 0) {
      Issuer m{sm, tmem, 1, 0, 0, 0, 0, true};
      if (a.do_post) {
        m.mlp_second(lo_post & 4, n_mine, D);
        // this CTA's second GEMM is complete once these MMAs are: its second weight ring and hidden
        // operand buffers are then free to receive the peer's partial sums, and the peer is told so
        // by the tensor core itself
        if (csize > 1) umma_commit_addr(map_to_rank(smem_u32(&sm->x_ready), crank ^ 1u));
      }
      if (a.do_head) m.mlp_second(a.tc_head_lo & 2, h_mine, 16);
    }
  } else {
    // ---------------------------------- epilogue ----------------------------------
    Epilogue<D> e;
    constexpr int PART = Epilogue<D>::PART;
#ifdef ARTAB_TIMELINE
    const bool tl_on = threadIdx.x == 64;
    e.tl_slot = a.tl_slot;
#endif
    TL(0);
    e.sm = sm;
    e.row = 32 * (warp & 3) + lane;
    e.wg = (warp - 2) >> 2;
    e.col0 = e.wg * PART;
    e.t_row = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
    e.acc_phase = e.xs_phase = 0;
    e.h_count = e.free_count = 0;
    e.ok = true;
    const long grow = row0 + e.row;
    const bool valid = grow < a.rows;
    const size_t goff = (size_t)grow * D + e.col0;
    float v[PART];

    // lane-major workspaces (attn, x1): a warp's 32 rows form one contiguous 512-byte span per float4;
    // the workspaces are padded to whole 128-row tiles, so no row guard is needed
    const size_t lm0 = lane_major_index(grow, e.col0, D);
    auto load_lm = [&](const float* src) {
#pragma unroll
      for (int i = 0; i < PART; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(src + lm0 + (size_t)(i >> 2) * 128);
        v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
      }
    };
    auto store_lm = [&](float* dst) {
#pragma unroll
      for (int i = 0; i < PART; i += 4)
        *reinterpret_cast<float4*>(dst + lm0 + (size_t)(i >> 2) * 128) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    };
    // row-major workspace (x, z): each thread touches its own contiguous slice
    auto load_row = [&](const float* src) {
#pragma unroll
      for (int i = 0; i < PART; i += 4) {
        const float4 t = valid ? *reinterpret_cast<const float4*>(src + goff + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
      }
    };
    auto store_row = [&](float* dst) {
      if (!valid) return;
#pragma unroll
      for (int i = 0; i < PART; i += 4)
        *reinterpret_cast<float4*>(dst + goff + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    };

    // Small per-column vectors -> shared memory (read by every epilogue thread, many times): the values
    // were fetched at the top of the kernel, so their latency is behind us by now.
    {
      const int i = threadIdx.x - 64;
      if (i < D) {
#pragma unroll
        for (int k = 0; k < 7; ++k) sm->vec[k][i] = cv[k];
      }
      if (a.do_post) {
#pragma unroll
        for (int k = 0; k < kBiasPerThread; ++k)
          if (i + k * kEpi < a.Dff) sm->bias_h[i + k * kEpi] = cb[k];
      }
    }
    // Everything above (and the weight producers' first tiles) needed nothing from the preceding
    // kernel; the activations do.
    TL(1);
    dep_wait();
    dep_trigger();
    TL(2);
    TLG(30);
    TLS(1);
    if (a.do_post) {
      load_lm(a.attn);
      e.publish_ax(v);
      TL(3);
      if (csize > 1) {  // free here (the first GEMM runs): the peer's barriers are known to exist from now on
        cluster_wait();
        cluster_waited = true;
      }
      load_lm(a.x1_in);                          // residual
      e.wait_acc();
      TL(4);
      e.sync_groups();                           // the staged vectors are complete
      e.add_acc(v);
      e.layer_norm(v, sm->vec[0], sm->vec[1]);   // v = x2
      TL(25);
      e.publish_ax(v);
      TL(5);
      // x2 is the residual of the last LayerNorm.  The MLP epilogue needs the registers, and x2 sits in
      // tensor memory anyway as the hi + lo operand just published: it is read back from there.
      TL(6);
      {
        int jl = 0;
        for (int j = crank; j < nt; j += csize, ++jl) {
          e.hidden_tile(jl, j, sm->bias_h);
          TL(7 + (jl < 5 ? jl : 5));
        }
      }
      e.wait_acc();
      e.drain_free();
      TL(13);
      if (csize > 1) e.send_partial(crank ^ 1u);   // the own partial sums travel while the lines below run
      e.load_ax(v);
#pragma unroll
      for (int i = 0; i < PART; i += 4) {
        const float4 b = *reinterpret_cast<const float4*>(&sm->vec[2][e.col0 + i]);
        v[i] += b.x; v[i + 1] += b.y; v[i + 2] += b.z; v[i + 3] += b.w;
      }
      if (csize > 1)
        e.receive_add(v);
      else
        e.add_acc(v);
      TL(14);
      e.layer_norm(v, sm->vec[3], sm->vec[4]);   // v = x3
      if (a.x_out && crank == 0) store_row(a.x_out);
      TL(15);
    } else {
      if (a.x_in_lane_major) load_lm(a.x_in); else load_row(a.x_in);
      e.sync_groups();                           // the staged vectors are complete
    }
    if (a.do_final) {
      e.quadrant_sync();                                       // the previous LayerNorm's statistics have been read
      e.layer_norm(v, sm->vec[5], sm->vec[6]);                 // v = z
      if (a.z_out && crank == 0) store_row(a.z_out);
    }
    if (a.do_head) {
      // the hidden bias buffer now takes the head's first-layer bias (every thread is past the MLP)
      e.sync_groups();
      {
        float bh[(1024 + kEpi - 1) / kEpi];
#pragma unroll
        for (int k = 0; k < (1024 + kEpi - 1) / kEpi; ++k) {
          const int i = threadIdx.x - 64 + k * kEpi;
          bh[k] = i < a.Dff ? __ldg(a.ba + i) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < (1024 + kEpi - 1) / kEpi; ++k) {
          const int i = threadIdx.x - 64 + k * kEpi;
          if (i < a.Dff) sm->bias_h[i] = bh[k];
        }
      }
      e.sync_groups();
      e.publish_ax(v);
      {
        int jl = 0;
        for (int j = h_first; j < nt; j += h_step, ++jl) e.hidden_tile(jl, j, sm->bias_h);
      }
      e.wait_acc();
      e.drain_free();
      TL(24);
      // 16 raw head outputs per row, held by the first column group; a pair adds its two partials
      // (second exchange of the launch: slots 2 and 3 of the scratch, barrier phase 1)
      uint32_t r[16];
      float peer_raw[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) peer_raw[i] = 0.f;
      if (e.wg == 0) {
        tmem_ld16(e.t_row + kAccA, r);
        tmem_wait_ld();
      }
      if (head_pair) {
        if (!cluster_waited) {  // a launch whose first remote access is this one
          cluster_wait();
          cluster_waited = true;
        }
        float* mine = a.pair_scratch + (size_t)(2 + crank) * a.pair_slot_stride + (size_t)grow * 16;
        const float* theirs = a.pair_scratch + (size_t)(2 + (crank ^ 1u)) * a.pair_slot_stride + (size_t)grow * 16;
        if (e.wg == 0) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            reinterpret_cast<uint4*>(mine)[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_rank(smem_u32(&sm->x_full), crank ^ 1u));
        e.ok = mbar_wait_cluster(&sm->x_full, a.do_post ? 1 : 0, &sm->abort_flag) && e.ok;
        if (e.wg == 0) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(theirs) + q);
            peer_raw[4 * q] = t.x; peer_raw[4 * q + 1] = t.y; peer_raw[4 * q + 2] = t.z; peer_raw[4 * q + 3] = t.w;
          }
        }
      }
      if (e.wg == 0) {
        float raw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          raw[i] = (__uint_as_float(r[i]) + peer_raw[i]) + (i < 3 * a.n_comp ? __ldg(a.bb + i) : 0.f);
        if (valid && e.ok && crank == 0) head_row_thread(a, raw, grow);
      }
    } else if (a.do_pre) {
      e.publish_ax(v);
      TL(16);
      e.wait_acc();
      TL(17);
      e.add_acc(v);
      e.layer_norm(v, sm->vec[5], sm->vec[6]);     // v = x1
      e.publish_ax(v);       // the Q projection's MMAs start on this
      TL(18);
      store_lm(a.x1_out);    // ... while the residual for the next launch drains to memory
      // q, k, v projections, one accumulator round each.  Destinations of this row's K / V are
      // resolved once (no per-element division): context cache rows during prefill, the private
      // buffer slot (in-place append) otherwise.
      const int Dh = a.kv.head_dim;
      const int dh_shift = Dh == 16 ? 4 : (Dh == 32 ? 5 : 6);
      __nv_bfloat16* k_dst = nullptr;   // element (h, d) at k_dst + h * k_hstride + d
      __nv_bfloat16* v_dst = nullptr;   // buffer / fp-layout V: v_dst + h * k_hstride + d
      __nv_bfloat16* vt_dst = nullptr;  // transposed hi|lo context V: vt_dst + (h * 2 * Dh + d) * Ncp
      size_t k_hstride = 0;
      if (valid && a.kv.mode == KV_PREFILL) {
        const long g = grow / a.kv.n_ctx, i = grow - g * a.kv.n_ctx;
        k_hstride = (size_t)a.kv.n_ctx_pad * Dh;
        k_dst = reinterpret_cast<__nv_bfloat16*>(a.kv.k_ctx) + ((size_t)g * a.kv.n_heads * a.kv.n_ctx_pad + i) * Dh;
        vt_dst = reinterpret_cast<__nv_bfloat16*>(a.kv.v_ctx) + (size_t)g * a.kv.n_heads * 2 * Dh * a.kv.n_ctx_pad + i;
      } else if (valid && (a.kv.mode == KV_DECODE || a.kv.mode == KV_TF)) {
        const long b = grow / a.kv.tokens_per_stream;
        const int j = (int)(grow - b * a.kv.tokens_per_stream);
        if (j < a.kv.n_kv_tokens) {
          k_hstride = (size_t)a.kv.max_buf * 2 * Dh;
          k_dst = reinterpret_cast<__nv_bfloat16*>(a.kv.kv_buf) +
                  ((size_t)b * a.kv.n_heads * a.kv.max_buf + a.kv.pos0 + j) * 2 * Dh;
          v_dst = k_dst + Dh;
        }
      }
      if (e.wg == 0) sm->rowdst[e.row] = direct_mode(a.kv.mode) ? nullptr : k_dst;
      // Staging tile for coalesced stores: [128 rows][D bf16] with 16 bytes of padding per row
      // (conflict-free 16-byte accesses), in the hidden-operand buffer, which is idle in this phase.
      constexpr int kStageRow = D * 2 + 16;
      uint8_t* stage = &sm->ah[0][0][0];
      // K / V go straight from registers to the cache during prefill (context cache: a row's store is
      // already a coalesced span) and in a decode step (one buffer row per stream: 16-byte pieces that
      // no staging could merge); teacher forcing stages them (consecutive positions of a stream)
      const bool direct = a.kv.mode == KV_PREFILL || a.kv.mode == KV_DECODE;
      const int tid_e = threadIdx.x - 64;
      for (int t = t_begin; t < t_end; ++t) {
        e.wait_acc();
        TL(20 + 2 * (t - t_begin));
        uint32_t r[Epilogue<D>::NCH][16];
#pragma unroll
        for (int c = 0; c < Epilogue<D>::NCH; ++c) tmem_ld16(e.t_row + kAccA + e.col0 + 16 * c, r[c]);
        tmem_wait_ld();
        if (t + 1 < t_end) {  // the accumulator is in registers: the next projection may overwrite it
          tc_fence_before();
          mbar_arrive(&sm->ep_done);
        }
        if (t == 0 || !direct) {
          // bf16 -> staging tile
#pragma unroll
          for (int c = 0; c < Epilogue<D>::NCH; ++c) {
            uint32_t pk[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              pk[i] = pack_bf16(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
            uint4* dst = reinterpret_cast<uint4*>(stage + (size_t)e.row * kStageRow + (e.col0 + 16 * c) * 2);
            dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
          e.sync_groups();
          constexpr int kChunksPerRow = D / 8;  // 16-byte chunks
          if (t == 0) {
            // q rows of this tile are one contiguous block of global memory
            __nv_bfloat16* qdst = reinterpret_cast<__nv_bfloat16*>(a.q_out) + (size_t)row0 * D;
            const int n_rows = (int)min((long)BM, (long)a.rows - row0);
            for (int idx = tid_e; idx < n_rows * kChunksPerRow; idx += kEpi) {
              const int rr = idx / kChunksPerRow, ch = idx - rr * kChunksPerRow;
              *reinterpret_cast<uint4*>(qdst + (size_t)idx * 8) =
                  *reinterpret_cast<const uint4*>(stage + (size_t)rr * kStageRow + ch * 16);
            }
          } else if (a.kv.mode == KV_DECODE || a.kv.mode == KV_TF) {
            // K (t = 1) or V (t = 2) of the buffer tokens: 16-byte chunks, Dh / 8 lanes per (row, head)
            const int cph_shift = dh_shift - 3;  // 16-byte chunks per head = Dh / 8
            const size_t hstride = (size_t)a.kv.max_buf * 2 * Dh;
            for (int idx = tid_e; idx < BM * kChunksPerRow; idx += kEpi) {
              const int rr = idx / kChunksPerRow, ch = idx - rr * kChunksPerRow;
              __nv_bfloat16* base = sm->rowdst[rr];
              if (!base) continue;
              const int hh = ch >> cph_shift, cc = ch & ((1 << cph_shift) - 1);
              *reinterpret_cast<uint4*>(base + hh * hstride + (t - 1) * Dh + cc * 8) =
                  *reinterpret_cast<const uint4*>(stage + (size_t)rr * kStageRow + ch * 16);
            }
          }
          e.sync_groups();  // the staging tile is reused by the next projection
          TL(21 + 2 * (t - t_begin));
        } else {
          // prefill: context K rows and the transposed hi|lo context V, written straight from registers
#pragma unroll
          for (int c = 0; c < Epilogue<D>::NCH; ++c) {
            const int cbase = e.col0 + 16 * c;
            if (t == 1 && k_dst) {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int col = cbase + 8 * i;
                const int h = col >> dh_shift, d = col & (Dh - 1);
                *reinterpret_cast<uint4*>(k_dst + (size_t)h * k_hstride + d) = make_uint4(
                    pack_bf16(__uint_as_float(r[c][8 * i]), __uint_as_float(r[c][8 * i + 1])),
                    pack_bf16(__uint_as_float(r[c][8 * i + 2]), __uint_as_float(r[c][8 * i + 3])),
                    pack_bf16(__uint_as_float(r[c][8 * i + 4]), __uint_as_float(r[c][8 * i + 5])),
                    pack_bf16(__uint_as_float(r[c][8 * i + 6]), __uint_as_float(r[c][8 * i + 7])));
              }
            } else if (t == 2 && v_dst) {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int col = cbase + 8 * i;
                const int h = col >> dh_shift, d = col & (Dh - 1);
                *reinterpret_cast<uint4*>(v_dst + (size_t)h * k_hstride + d) = make_uint4(
                    pack_bf16(__uint_as_float(r[c][8 * i]), __uint_as_float(r[c][8 * i + 1])),
                    pack_bf16(__uint_as_float(r[c][8 * i + 2]), __uint_as_float(r[c][8 * i + 3])),
                    pack_bf16(__uint_as_float(r[c][8 * i + 4]), __uint_as_float(r[c][8 * i + 5])),
                    pack_bf16(__uint_as_float(r[c][8 * i + 6]), __uint_as_float(r[c][8 * i + 7])));
              }
            } else if (t == 2 && vt_dst) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int col = cbase + i;
                const int h = col >> dh_shift, d = col & (Dh - 1);
                const float val = __uint_as_float(r[c][i]);
                const __nv_bfloat16 hi = __float2bfloat16_rn(val);
                __nv_bfloat16* p = vt_dst + ((size_t)h * 2 * Dh + d) * a.kv.n_ctx_pad;
                p[0] = hi;
                p[(size_t)Dh * a.kv.n_ctx_pad] = __float2bfloat16_rn(val - __bfloat162float(hi));
              }
            }
          }
        }
      }
    }
    if (!e.ok && threadIdx.x == 64 && a.status) atomicExch(a.status, 3);
    TL(26);
    TLG(31);
    TLS(2);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (csize > 1) {
    if (!cluster_waited) cluster_wait();
    cluster_sync_all();  // neither CTA leaves while the other could still address its shared memory
  }
  if (threadIdx.x == 64) ARTAB_STAMP(1, 3);
}

}  // namespace


bool dense_tc_applicable(const DenseArgs& a) {
  if (a.kv.dtype != ARTAB_BF16) return false;
  if (!(a.D == 64 || a.D == 128 || a.D == 192) || a.Dff % HT != 0 || a.Dff > 1024 || 3 * a.n_comp > 16 || a.n_comp > 8) return false;
  if (a.do_post && !(a.post_w.tc_wo && a.post_w.tc_w1 && a.post_w.tc_w2)) return false;
  if (a.do_pre && !(a.pre_w.tc_wf && a.pre_w.tc_wqkv)) return false;
  if (a.do_head && !(a.tc_wa && a.tc_wb)) return false;
  if (!a.do_post && !a.do_pre && !a.do_head) return false;
  return true;
}

int launch_dense_tc(const DenseArgs& a, cudaStream_t s) {
  if (a.rows <= 0) return ARTAB_OK;
  ARTAB_REQUIRE(dense_tc_applicable(a), ARTAB_EINVAL, "tensor-core dense chain: unsupported shape or missing tiles");
  const size_t smem = sizeof(Smem) + 1024;
  const int tiles = (a.rows + BM - 1) / BM;
  // Few row tiles (a decode step): the chain's latency is what counts, so a CTA pair shares each
  // tile.  Many tiles (prefill, teacher forcing): one CTA per tile keeps every SM on its own rows.
  static const bool allow_pair = !(getenv("ARTAB_DENSE_PAIR") && getenv("ARTAB_DENSE_PAIR")[0] == '0');
  const unsigned csize =
      (allow_pair && a.pair_scratch && a.pair_slots >= 6 && 2 * tiles <= kPairMaxCtas && a.Dff / HT >= 2) ? 2u : 1u;
  const int grid = tiles * (int)csize;
  cudaError_t e = cudaSuccess;
  static SmemConfig configured[3];
#ifdef ARTAB_TIMELINE
  static int tl_next = 0;
  const_cast<DenseArgs&>(a).tl_slot = tl_next++ & 31;
  ARTAB_STAMP_ATTACH();
#endif
  prof_begin(PROF_DENSE, s);
  switch (a.D) {
    case 64:
      e = configured[0].ensure(dense_tc_kernel<64>, smem);
      if (e == cudaSuccess) e = launch_dependent_cluster(dense_tc_kernel<64>, dim3(grid), dim3(kThreads), smem, s, csize, a);
      break;
    case 128:
      e = configured[1].ensure(dense_tc_kernel<128>, smem);
      if (e == cudaSuccess) e = launch_dependent_cluster(dense_tc_kernel<128>, dim3(grid), dim3(kThreads), smem, s, csize, a);
      break;
    default:
      e = configured[2].ensure(dense_tc_kernel<192>, smem);
      if (e == cudaSuccess) e = launch_dependent_cluster(dense_tc_kernel<192>, dim3(grid), dim3(kThreads), smem, s, csize, a);
      break;
  }
  prof_end(s);
  ARTAB_REQUIRE(e == cudaSuccess, ARTAB_ELAUNCH, "dense_tc_kernel: launch refused: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("dense_tc_kernel");
}

}  // namespace artab

#ifdef ARTAB_TIMELINE
// diagnostic builds: copy the timeline stamps [32 launch slots][32 CTAs][32 marks] to host memory
extern "C" __attribute__((visibility("default"))) int artab_debug_timeline(long long* host_dst) {
  return (int)cudaMemcpyFromSymbol(host_dst, artab::g_tl, sizeof(long long) * 32 * 32 * 32);
}
#endif
