// C ABI of libartab_b200.so: argument checking, kernel sequencing of the whole
// path (prefill, decode step, teacher forcing) and the single-operator entry
// points.  Nothing here allocates or synchronises.
#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "attn.cuh"
#include "dense.cuh"

namespace artab {

static thread_local char g_err[512] = "";
static thread_local int64_t g_launches = 0;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// ---- optional per-launch timing (benchmarks) -----------------------------------
// When enabled, every kernel launch of this library is bracketed by a pair of CUDA
// events on the launching stream; artab_profile_read sums the elapsed time per
// kernel kind after the caller has synchronised.  Off by default: no events.
struct ProfSlot {
  cudaEvent_t a, b;
  int kind;
};
static thread_local bool g_prof_on = false;
static thread_local std::vector<ProfSlot>* g_prof = nullptr;
static thread_local std::vector<ProfSlot>* g_prof_pool = nullptr;

void count_launch() { ++g_launches; }

// On unless the environment says ARTAB_DEPENDENT_LAUNCH=0 (profilers that replay single kernels
// want plain launches) or artab_set_dependent_launch(0) is called.
static int dependent_launch_default() {
  const char* e = getenv("ARTAB_DEPENDENT_LAUNCH");
  return !(e && e[0] == '0');
}
static std::atomic<int> g_dependent_launch{dependent_launch_default()};
static std::atomic<long long> g_debug_wait_cycles{0};
static std::atomic<int> g_debug_drop_score_commits{0};
long long debug_wait_cycles() { return g_debug_wait_cycles.load(std::memory_order_relaxed); }
int debug_drop_score_commits() { return g_debug_drop_score_commits.load(std::memory_order_relaxed); }

static thread_local int g_plain_scope = 0;
PlainLaunchScope::PlainLaunchScope() { ++g_plain_scope; }
PlainLaunchScope::~PlainLaunchScope() { --g_plain_scope; }
bool dependent_launch_enabled() {
  return g_plain_scope == 0 && g_dependent_launch.load(std::memory_order_relaxed) != 0;
}

void prof_begin(int kind, cudaStream_t s) {
  if (!g_prof_on) return;
  if (!g_prof) g_prof = new std::vector<ProfSlot>();
  if (!g_prof_pool) g_prof_pool = new std::vector<ProfSlot>();
  ProfSlot sl;
  if (!g_prof_pool->empty()) {
    sl = g_prof_pool->back();
    g_prof_pool->pop_back();
  } else {
    cudaEventCreate(&sl.a);
    cudaEventCreate(&sl.b);
  }
  sl.kind = kind;
  cudaEventRecord(sl.a, s);
  g_prof->push_back(sl);
}

void prof_end(cudaStream_t s) {
  if (!g_prof_on || !g_prof || g_prof->empty()) return;
  cudaEventRecord(g_prof->back().b, s);
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();  // reads and clears: one failed launch does not poison later calls
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return ARTAB_ELAUNCH;
  }
  return ARTAB_OK;
}

namespace {

constexpr int kSMs = 148;
constexpr int kMaxSplits = 16;

inline size_t esize(int dtype) { return dtype == ARTAB_BF16 ? 2 : 4; }

int check_model(const artab_model* m) {
  ARTAB_REQUIRE(m && m->layers, ARTAB_EINVAL, "model: null");
  ARTAB_REQUIRE(m->n_heads > 0 && m->head_dim * m->n_heads == m->d_model, ARTAB_EINVAL,
                "model: d_model %d != n_heads %d * head_dim %d", m->d_model, m->n_heads, m->head_dim);
  ARTAB_REQUIRE(m->head_dim == 16 || m->head_dim == 32 || m->head_dim == 64, ARTAB_EINVAL,
                "model: head_dim %d not supported (16, 32, 64)", m->head_dim);
  ARTAB_REQUIRE(m->n_layers >= 1 && m->n_comp >= 2 && m->n_ar_tokens >= 1, ARTAB_EINVAL, "model: bad sizes");
  return ARTAB_OK;
}

int check_state(const artab_model* m, const artab_state* st) {
  ARTAB_REQUIRE(st, ARTAB_EINVAL, "state: null");
  ARTAB_REQUIRE(st->dtype == ARTAB_F32 || st->dtype == ARTAB_BF16, ARTAB_EINVAL, "state: bad dtype %d", st->dtype);
  ARTAB_REQUIRE(st->n_groups == 1 || st->n_groups == st->n_streams, ARTAB_EINVAL,
                "state: n_groups must be 1 (shared context) or n_streams");
  ARTAB_REQUIRE(st->n_ctx > 0 && st->n_ctx_pad >= st->n_ctx && st->n_ctx_pad % 8 == 0, ARTAB_EINVAL,
                "state: n_ctx %d / n_ctx_pad %d (pad must be a multiple of 8)", st->n_ctx, st->n_ctx_pad);
  ARTAB_REQUIRE(st->k_ctx && st->v_ctx && st->x && st->x1 && st->attn && st->q && st->o_part && st->lse_part,
                ARTAB_EINVAL, "state: null buffer");
  ARTAB_REQUIRE(st->max_splits >= 1, ARTAB_EINVAL, "state: max_splits < 1");
  ARTAB_REQUIRE(st->max_rows % 128 == 0, ARTAB_EINVAL, "state: max_rows must be a multiple of 128");
  (void)m;
  return ARTAB_OK;
}

struct Layout {
  size_t ctx_layer, vctx_layer, buf_layer;  // elements per layer
};

Layout layout_of(const artab_model* m, const artab_state* st) {
  Layout l;
  l.ctx_layer = (size_t)st->n_groups * m->n_heads * st->n_ctx_pad * m->head_dim;
  l.vctx_layer = l.ctx_layer * (st->dtype == ARTAB_BF16 ? 2 : 1);  // bf16 V: hi and lo parts
  l.buf_layer = (size_t)st->n_streams * m->n_heads * st->max_buf * 2 * m->head_dim;
  return l;
}

inline void* off(void* p, size_t elems, int dtype) { return (char*)p + elems * esize(dtype); }

bool use_tc(int dtype, int head_dim) { return ctx_attn_tc_supported(dtype, head_dim); }

int plan_splits(int dtype, int head_dim, int rows, int rows_per_group, int n_groups, int n_heads, int n_ctx,
                int max_splits) {
  const bool tc = use_tc(dtype, head_dim);
  const int tile_m = tc ? 128 : 16, tile_k = tc ? 128 : 64;
  const int rows_g = n_groups == 1 ? rows : rows_per_group;
  const long items = (long)((rows_g + tile_m - 1) / tile_m) * n_heads * n_groups;
  const int tiles = (n_ctx + tile_k - 1) / tile_k;
  // Resident CTA slots: two per SM for the tensor-core kernel (TMEM), about eight for the SIMT one.
  const long slots = (long)kSMs * (tc ? 2 : 8);
  // Cost model: waves x (key tiles per CTA + fixed per-CTA overhead in tile units); smallest wins.
  int best = 1;
  double best_cost = 1e30;
  const int smax = tiles < max_splits ? tiles : max_splits;
  for (int s = 1; s <= smax; ++s) {
    const int tps = (tiles + s - 1) / s;
    const int s_eff = (tiles + tps - 1) / tps;
    if (s_eff != s) continue;
    const long waves = (items * s + slots - 1) / slots;
    const double cost = (double)waves * (tps + 1.5) + 0.05 * s;  // small bias against extra partials
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// The tensor-core chain reads attn / x1 in the lane-major layout (workspaces padded to 128 rows).
bool chain_on_tc(const artab_model* m, const artab_state* st) {
  if (st->dtype != ARTAB_BF16 || !m->tc_wa || !m->tc_wb) return false;
  for (int l = 0; l < m->n_layers; ++l)
    if (!m->layers[l].tc_wo || !m->layers[l].tc_w1 || !m->layers[l].tc_w2 || !m->layers[l].tc_wf ||
        !m->layers[l].tc_wqkv)
      return false;
  DenseArgs probe;
  memset(&probe, 0, sizeof(probe));
  probe.D = m->d_model;
  probe.Dff = m->d_ff;
  probe.n_comp = m->n_comp;
  probe.kv.dtype = st->dtype;
  probe.do_head = 1;
  probe.tc_wa = m->tc_wa;
  probe.tc_wb = m->tc_wb;
  return dense_tc_applicable(probe);
}

int run_ctx(const artab_model* m, const artab_state* st, int layer, int rows, int rows_per_group, int n_splits,
            float* out, float* lse, bool kv_stable, cudaStream_t s) {
  const Layout lo = layout_of(m, st);
  CtxAttnArgs c;
  memset(&c, 0, sizeof(c));
  c.dtype = st->dtype;
  c.q = st->q;
  c.k_ctx = off(st->k_ctx, lo.ctx_layer * layer, st->dtype);
  c.v_ctx = off(st->v_ctx, lo.vctx_layer * layer, st->dtype);
  c.v_transposed = st->dtype == ARTAB_BF16;
  c.rows = rows;
  c.rows_per_group = rows_per_group;
  c.n_groups = st->n_groups;
  c.n_heads = m->n_heads;
  c.head_dim = m->head_dim;
  c.n_ctx = st->n_ctx;
  c.n_ctx_pad = st->n_ctx_pad;
  c.n_splits = n_splits;
  c.scale = 1.0f / sqrtf((float)m->head_dim);
  c.out = out;
  c.out_lane_major = out == st->attn && chain_on_tc(m, st);
  c.lse = lse;
  c.status = st->status;
  c.kv_stable = kv_stable ? 1 : 0;
  return use_tc(st->dtype, m->head_dim) ? launch_ctx_attn_tc(c, s) : launch_ctx_attn_simt(c, s);
}

void fill_head(const artab_model* m, DenseArgs& d) {
  d.lnf_g = m->lnf_g;
  d.lnf_b = m->lnf_b;
  d.wa_t = m->wa_t;
  d.ba = m->ba;
  d.wb_t = m->wb_t;
  d.bb = m->bb;
  d.mean_bias = m->mean_bias;
  d.std_bias = m->std_bias;
  d.weight_bias = m->weight_bias;
  d.tc_wa = m->tc_wa;
  d.tc_wb = m->tc_wb;
  d.tc_head_lo = m->tc_head_lo;
}

DenseArgs dense_base(const artab_model* m, const artab_state* st, int rows) {
  DenseArgs d;
  memset(&d, 0, sizeof(d));
  d.rows = rows;
  d.D = m->d_model;
  d.Dff = m->d_ff;
  d.n_comp = m->n_comp;
  d.attn = st->attn;
  d.x1_in = st->x1;
  d.x_in = st->x;
  d.x1_out = st->x1;
  d.q_out = st->q;
  d.kv.mode = KV_NONE;
  d.kv.dtype = st->dtype;
  d.kv.n_heads = m->n_heads;
  d.kv.head_dim = m->head_dim;
  d.status = st->status;
  d.lane_major = chain_on_tc(m, st);
  // the context-partial workspace is idle while a dense chain runs: its first two slots serve the
  // CTA pairs' exchange
  if (st->max_splits >= 6) {
    d.pair_scratch = st->o_part;
    d.pair_slot_stride = (size_t)st->max_rows * m->d_model;
    d.pair_slots = st->max_splits;
  }
  fill_head(m, d);
  return d;
}

void set_kv(const artab_model* m, const artab_state* st, int layer, KvDest& kv) {
  const Layout lo = layout_of(m, st);
  kv.k_ctx = off(st->k_ctx, lo.ctx_layer * layer, st->dtype);
  kv.v_ctx = off(st->v_ctx, lo.vctx_layer * layer, st->dtype);
  kv.n_ctx = st->n_ctx;
  kv.n_ctx_pad = st->n_ctx_pad;
  kv.kv_buf = st->kv_buf ? off(st->kv_buf, lo.buf_layer * layer, st->dtype) : nullptr;
  kv.max_buf = st->max_buf;
}

EmbedArgs embed_base(const artab_model* m) {
  EmbedArgs e;
  memset(&e, 0, sizeof(e));
  e.D = m->d_model;
  e.wx = m->wx;
  e.bx = m->bx;
  e.wy = m->wy;
  e.by = m->by;
  e.marker = m->marker;
  e.ar_tokens = m->ar_tokens;
  e.S = m->n_ar_tokens;
  return e;
}

// Layers of a decode-like pass (decode step or teacher forcing) after layer 0's
// "pre" stage has run.  `kv_proto` carries the scatter description for the next
// layer's pre stage; `last` describes what follows the last layer.
int run_layers(const artab_model* m, artab_state* st, int rows, int rows_per_group, const KvDest& kv_proto,
               const BufMergeArgs& buf_proto, bool need_merge, const DenseArgs& last, cudaStream_t s) {
  const Layout lo = layout_of(m, st);
  const int n_splits =
      plan_splits(st->dtype, m->head_dim, rows, rows_per_group, st->n_groups, m->n_heads, st->n_ctx, st->max_splits);
  for (int l = 0; l < m->n_layers; ++l) {
    int rc;
    if (!need_merge && n_splits == 1) {
      rc = run_ctx(m, st, l, rows, rows_per_group, 1, st->attn, st->lse_part, true, s);
      if (rc) return rc;
    } else {
      rc = run_ctx(m, st, l, rows, rows_per_group, n_splits, st->o_part, st->lse_part, true, s);
      if (rc) return rc;
      BufMergeArgs b = buf_proto;
      b.kv_buf = st->kv_buf ? off(st->kv_buf, lo.buf_layer * l, st->dtype) : nullptr;
      b.n_splits = n_splits;
      rc = launch_buf_merge(b, s);
      if (rc) return rc;
    }
    if (l + 1 < m->n_layers) {
      DenseArgs d = dense_base(m, st, rows);
      d.do_post = 1;
      d.do_pre = 1;
      d.post_w = m->layers[l];
      d.pre_w = m->layers[l + 1];
      d.kv = kv_proto;
      set_kv(m, st, l + 1, d.kv);
      rc = launch_dense(d, s);
    } else {
      DenseArgs d = last;
      d.post_w = m->layers[l];
      rc = launch_dense(d, s);
    }
    if (rc) return rc;
  }
  return ARTAB_OK;
}

BufMergeArgs buf_base(const artab_model* m, const artab_state* st, int rows) {
  BufMergeArgs b;
  memset(&b, 0, sizeof(b));
  b.dtype = st->dtype;
  b.q = st->q;
  b.n_heads = m->n_heads;
  b.head_dim = m->head_dim;
  b.max_buf = st->max_buf;
  b.o_part = st->o_part;
  b.lse_part = st->lse_part;
  b.rows = rows;
  b.scale = 1.0f / sqrtf((float)m->head_dim);
  b.out = st->attn;
  b.out_lane_major = chain_on_tc(m, st);
  return b;
}

int decode_common(const artab_model* m, artab_state* st, int n_new, const DenseArgs& last_proto, bool x_lane_major,
                  cudaStream_t s) {
  const int rows = st->n_streams * n_new;
  ARTAB_REQUIRE(rows <= st->max_rows, ARTAB_ECAPACITY, "decode: %d rows exceed the workspace (%d)", rows,
                st->max_rows);
  ARTAB_REQUIRE(st->buffer_len + (n_new - 1) <= st->max_buf && (n_new == 1 || st->kv_buf), ARTAB_ECAPACITY,
                "Shared-context buffer cache exceeded; increase max buffer length.");
  // layer 0 pre stage: LN1 + QKV + in-place append of the buffer token's K/V
  KvDest kv;
  memset(&kv, 0, sizeof(kv));
  kv.mode = KV_DECODE;
  kv.dtype = st->dtype;
  kv.n_heads = m->n_heads;
  kv.head_dim = m->head_dim;
  kv.tokens_per_stream = n_new;
  kv.n_kv_tokens = n_new - 1;
  kv.pos0 = st->buffer_len;
  DenseArgs d0 = dense_base(m, st, rows);
  d0.do_pre = 1;
  d0.pre_w = m->layers[0];
  d0.kv = kv;
  d0.x_in_lane_major = x_lane_major;
  set_kv(m, st, 0, d0.kv);
  int rc = launch_dense(d0, s);
  if (rc) return rc;

  const int len = st->buffer_len + (n_new - 1);
  BufMergeArgs b = buf_base(m, st, rows);
  b.mode_tf = 0;
  b.n_new = n_new;
  b.len0 = len;
  b.n_items = (long)st->n_streams * m->n_heads;
  DenseArgs last = last_proto;
  last.rows = rows;
  return run_layers(m, st, rows, n_new, kv, b, /*need_merge=*/len > 0, last, s);
}

}  // namespace
}  // namespace artab

using namespace artab;

#ifdef ARTAB_TIMELINE
// diagnostic builds: the stamp log shared by all kernels (see common.cuh) and its reader
namespace artab {
StampLog* stamp_log_buffer() {
  static StampLog* buf = nullptr;
  if (!buf && cudaMalloc(&buf, sizeof(StampLog)) == cudaSuccess) cudaMemset(buf, 0, sizeof(StampLog));
  return buf;
}
}  // namespace artab
#endif

extern "C" {

int artab_plan_splits(int dtype, int rows, int rows_per_group, int n_groups, int n_heads, int n_ctx) {
  return plan_splits(dtype, 32, rows, rows_per_group, n_groups, n_heads, n_ctx, kMaxSplits);
}

void artab_profile_enable(int on) { g_prof_on = on != 0; }

int artab_debug_set(int key, long long value) {
  switch (key) {
    case ARTAB_DEBUG_WAIT_CYCLES:
      ARTAB_REQUIRE(value >= 0, ARTAB_EINVAL, "debug_set: the wait limit must be >= 0 cycles");
      g_debug_wait_cycles.store(value, std::memory_order_relaxed);
      return ARTAB_OK;
    case ARTAB_DEBUG_DROP_SCORE_COMMITS:
      g_debug_drop_score_commits.store(value != 0, std::memory_order_relaxed);
      return ARTAB_OK;
    default:
      set_error("debug_set: unknown key %d", key);
      return ARTAB_EINVAL;
  }
}

#ifdef ARTAB_TIMELINE
// copies up to max_records (kernel * 10000 + event * 1000 + CTA (999: the last of a large grid), nanoseconds)
// pairs, empties the log and returns how many were copied
ARTAB_API long long artab_debug_stamps(long long* host_dst, long long max_records) {
  artab::StampLog* buf = artab::stamp_log_buffer();
  if (!buf || cudaDeviceSynchronize() != cudaSuccess) return -1;
  unsigned long long n = 0;
  if (cudaMemcpy(&n, &buf->n, sizeof n, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (n > (1ULL << 16)) n = 1ULL << 16;
  if ((long long)n > max_records) n = (unsigned long long)max_records;
  if (n && cudaMemcpy(host_dst, buf->rec, n * 2 * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  cudaMemset(&buf->n, 0, sizeof n);
  return (long long)n;
}
#endif

void artab_set_dependent_launch(int on) { g_dependent_launch.store(on != 0, std::memory_order_relaxed); }

int artab_profile_read(double* ms_per_kind, int64_t* launches_per_kind, int n_kinds) {
  for (int i = 0; i < n_kinds; ++i) {
    ms_per_kind[i] = 0.0;
    launches_per_kind[i] = 0;
  }
  if (!g_prof) return 0;
  int n = 0;
  for (ProfSlot& sl : *g_prof) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, sl.a, sl.b) == cudaSuccess && sl.kind >= 0 && sl.kind < n_kinds) {
      ms_per_kind[sl.kind] += ms;
      launches_per_kind[sl.kind] += 1;
      ++n;
    }
    g_prof_pool->push_back(sl);
  }
  g_prof->clear();
  return n;
}

int64_t artab_launch_count(void) { return g_launches; }
void artab_launch_count_reset(void) { g_launches = 0; }
const char* artab_last_error(void) { return g_err; }
const char* artab_version(void) { return "artab-b200 sm_100a"; }

int artab_prefill(const artab_model* m, artab_state* st, const float* xc, const float* yc, int n_feat,
                  void* stream) {
  int rc = check_model(m);
  if (rc) return rc;
  rc = check_state(m, st);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int rows = st->n_groups * st->n_ctx;
  ARTAB_REQUIRE(rows <= st->max_rows, ARTAB_ECAPACITY, "prefill: %d rows exceed the workspace (%d)", rows,
                st->max_rows);
  ARTAB_REQUIRE(xc && yc && n_feat > 0, ARTAB_EINVAL, "prefill: null input");
  EmbedArgs e = embed_base(m);
  e.mode = EMB_ROWS;
  e.rows = rows;
  e.F = n_feat;
  e.kind = ARTAB_MARK_CONTEXT;
  e.x = xc;
  e.y = yc;
  e.out = st->x;
  e.out_lane_major = chain_on_tc(m, st);
  rc = launch_embed(e, s);
  if (rc) return rc;

  KvDest kv;
  memset(&kv, 0, sizeof(kv));
  kv.mode = KV_PREFILL;
  kv.dtype = st->dtype;
  kv.n_heads = m->n_heads;
  kv.head_dim = m->head_dim;
  DenseArgs d0 = dense_base(m, st, rows);
  d0.do_pre = 1;
  d0.pre_w = m->layers[0];
  d0.kv = kv;
  d0.x_in_lane_major = chain_on_tc(m, st);   // written by the embedder above
  set_kv(m, st, 0, d0.kv);
  rc = launch_dense(d0, s);
  if (rc) return rc;
  for (int l = 0; l + 1 < m->n_layers; ++l) {
    // dense non-causal self-attention over the context rows of each group
    rc = run_ctx(m, st, l, rows, st->n_ctx, 1, st->attn, st->lse_part, false, s);
    if (rc) return rc;
    DenseArgs d = dense_base(m, st, rows);
    d.do_post = 1;
    d.do_pre = 1;
    d.post_w = m->layers[l];
    d.pre_w = m->layers[l + 1];
    d.kv = kv;
    set_kv(m, st, l + 1, d.kv);
    rc = launch_dense(d, s);
    if (rc) return rc;
  }
  // the last layer's attention and MLP feed nothing: only its K/V (written above) are kept
  st->buffer_len = 0;
  return ARTAB_OK;
}

int artab_decode_step(const artab_model* m, artab_state* st, const float* xt, int n_feat, int n_targets, int t,
                      float* samples, const float* expo, const float* normal, float* logdens, int32_t* comp,
                      void* stream) {
  int rc = check_model(m);
  if (rc) return rc;
  rc = check_state(m, st);
  if (rc) return rc;
  ARTAB_REQUIRE(xt && samples && expo && normal && t >= 0 && t < n_targets, ARTAB_EINVAL, "decode_step: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  const int n_new = t == 0 ? 1 : 2;
  const int rows = st->n_streams * n_new;
  ARTAB_REQUIRE(rows <= st->max_rows, ARTAB_ECAPACITY, "decode: %d rows exceed the workspace (%d)", rows,
                st->max_rows);
  EmbedArgs e = embed_base(m);
  e.mode = EMB_DECODE;
  e.rows = rows;
  e.F = n_feat;
  e.xt = xt;
  e.yt = samples;
  e.Nt = n_targets;
  e.t = t;
  e.n_new = n_new;
  e.out = st->x;
  e.out_lane_major = chain_on_tc(m, st);
  rc = launch_embed(e, s);
  if (rc) return rc;
  DenseArgs last = dense_base(m, st, rows);
  last.do_post = 1;
  last.do_final = 1;
  last.do_head = 1;
  last.head_mode = 1;
  last.head_tps = n_new;
  last.head_first = n_new - 1;
  last.out_stride = n_targets;
  last.out_col = t;
  last.expo = expo;
  last.normal = normal;
  last.y_out = samples;
  last.ld_out = logdens;
  last.comp_out = comp;
  rc = decode_common(m, st, n_new, last, chain_on_tc(m, st), s);
  if (rc) return rc;
  st->buffer_len += n_new - 1;
  return ARTAB_OK;
}

int artab_decode_embedded(const artab_model* m, artab_state* st, const float* x_in, int n_new, int commit,
                          float* z_out, void* stream) {
  int rc = check_model(m);
  if (rc) return rc;
  rc = check_state(m, st);
  if (rc) return rc;
  ARTAB_REQUIRE(n_new == 1 || n_new == 2, ARTAB_EINVAL,
                "Shared-context decode only supports N=1 (target) or N=2 (buffer, target).");
  ARTAB_REQUIRE(commit >= 0 && commit <= n_new - 1 && x_in && z_out, ARTAB_EINVAL, "decode_embedded: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  const int rows = st->n_streams * n_new;
  ARTAB_REQUIRE(rows <= st->max_rows, ARTAB_ECAPACITY, "decode: %d rows exceed the workspace (%d)", rows,
                st->max_rows);
  cudaError_t ce = cudaMemcpyAsync(st->x, x_in, (size_t)rows * m->d_model * sizeof(float), cudaMemcpyDeviceToDevice, s);
  ARTAB_REQUIRE(ce == cudaSuccess, ARTAB_ELAUNCH, "decode_embedded: copy failed: %s", cudaGetErrorString(ce));
  DenseArgs last = dense_base(m, st, rows);
  last.do_post = 1;
  last.do_final = 1;
  last.z_out = z_out;
  rc = decode_common(m, st, n_new, last, /*x_lane_major=*/false, s);
  if (rc) return rc;
  st->buffer_len += commit;
  return ARTAB_OK;
}

int artab_teacher_forcing(const artab_model* m, artab_state* st, const float* xt, const float* yt, int n_feat,
                          int n_targets, float* logdens, void* stream) {
  int rc = check_model(m);
  if (rc) return rc;
  rc = check_state(m, st);
  if (rc) return rc;
  ARTAB_REQUIRE(xt && yt && logdens && n_targets >= 1, ARTAB_EINVAL, "teacher_forcing: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  const int Nt = n_targets;
  const long rows_l = (long)st->n_streams * 2 * Nt;
  ARTAB_REQUIRE(rows_l <= st->max_rows, ARTAB_ECAPACITY, "teacher_forcing: %ld rows exceed the workspace (%d)", rows_l,
                st->max_rows);
  ARTAB_REQUIRE(Nt <= st->max_buf && st->kv_buf, ARTAB_ECAPACITY,
                "Shared-context buffer cache exceeded; increase max buffer length.");
  const int rows = (int)rows_l;
  EmbedArgs e = embed_base(m);
  e.mode = EMB_TF;
  e.rows = rows;
  e.F = n_feat;
  e.xt = xt;
  e.yt = yt;
  e.Nt = Nt;
  e.out = st->x;
  e.out_lane_major = chain_on_tc(m, st);
  rc = launch_embed(e, s);
  if (rc) return rc;
  KvDest kv;
  memset(&kv, 0, sizeof(kv));
  kv.mode = KV_TF;
  kv.dtype = st->dtype;
  kv.n_heads = m->n_heads;
  kv.head_dim = m->head_dim;
  kv.tokens_per_stream = 2 * Nt;
  kv.n_kv_tokens = Nt;
  kv.pos0 = 0;
  DenseArgs d0 = dense_base(m, st, rows);
  d0.do_pre = 1;
  d0.pre_w = m->layers[0];
  d0.kv = kv;
  d0.x_in_lane_major = chain_on_tc(m, st);   // written by the embedder above
  set_kv(m, st, 0, d0.kv);
  rc = launch_dense(d0, s);
  if (rc) return rc;
  BufMergeArgs b = buf_base(m, st, rows);
  b.mode_tf = 1;
  b.nt = Nt;
  b.n_items = (long)st->n_streams * m->n_heads * (Nt + 1);
  DenseArgs last = dense_base(m, st, rows);
  last.do_post = 1;
  last.do_final = 1;
  last.do_head = 1;
  last.head_mode = 2;
  last.head_tps = 2 * Nt;
  last.head_first = Nt;
  last.out_stride = Nt;
  last.out_col = 0;
  last.y_in = yt;
  last.ld_out = logdens;
  rc = run_layers(m, st, rows, 2 * Nt, kv, b, /*need_merge=*/true, last, s);
  if (rc) return rc;
  st->buffer_len = Nt;
  return ARTAB_OK;
}

int artab_forward_masked(const artab_model* m, artab_state* st, const float* xb, const float* yb, const float* xt,
                         const float* yt, int n_feat, int n_buf, int n_targets, const int32_t* visible,
                         float* logdens, void* stream) {
  int rc = check_model(m);
  if (rc) return rc;
  rc = check_state(m, st);
  if (rc) return rc;
  ARTAB_REQUIRE(xt && yt && logdens && visible && n_targets >= 1 && n_buf >= 0 && n_feat > 0, ARTAB_EINVAL,
                "forward_masked: bad argument");
  ARTAB_REQUIRE(n_buf == 0 || (xb && yb), ARTAB_EINVAL, "forward_masked: buffer rows without buffer inputs");
  ARTAB_REQUIRE(n_buf <= m->n_ar_tokens, ARTAB_EINVAL,
                "forward_masked: %d buffer rows but only %d AR position tokens", n_buf, m->n_ar_tokens);
  cudaStream_t s = (cudaStream_t)stream;
  const int tps = n_buf + n_targets;
  const long rows_l = (long)st->n_streams * tps;
  ARTAB_REQUIRE(rows_l <= st->max_rows, ARTAB_ECAPACITY, "forward_masked: %ld rows exceed the workspace (%d)", rows_l,
                st->max_rows);
  ARTAB_REQUIRE(n_buf == 0 || (n_buf <= st->max_buf && st->kv_buf), ARTAB_ECAPACITY,
                "Shared-context buffer cache exceeded; increase max buffer length.");
  const int rows = (int)rows_l;
  EmbedArgs e = embed_base(m);
  e.mode = EMB_FWD;
  e.rows = rows;
  e.F = n_feat;
  e.xb = xb;
  e.yb = yb;
  e.Nb = n_buf;
  e.xt = xt;
  e.Nt = n_targets;
  e.out = st->x;
  e.out_lane_major = chain_on_tc(m, st);
  rc = launch_embed(e, s);
  if (rc) return rc;
  KvDest kv;
  memset(&kv, 0, sizeof(kv));
  kv.mode = KV_TF;
  kv.dtype = st->dtype;
  kv.n_heads = m->n_heads;
  kv.head_dim = m->head_dim;
  kv.tokens_per_stream = tps;
  kv.n_kv_tokens = n_buf;
  kv.pos0 = 0;
  DenseArgs d0 = dense_base(m, st, rows);
  d0.do_pre = 1;
  d0.pre_w = m->layers[0];
  d0.kv = kv;
  d0.x_in_lane_major = chain_on_tc(m, st);   // written by the embedder above
  set_kv(m, st, 0, d0.kv);
  rc = launch_dense(d0, s);
  if (rc) return rc;
  BufMergeArgs b = buf_base(m, st, rows);
  b.mode_tf = 2;
  b.visible = visible;
  b.tps = tps;
  b.len0 = n_buf;  // upper bound of every visible count
  b.n_items = (long)st->n_streams * m->n_heads * tps;
  DenseArgs last = dense_base(m, st, rows);
  last.do_post = 1;
  last.do_final = 1;
  last.do_head = 1;
  last.head_mode = 2;
  last.head_tps = tps;
  last.head_first = n_buf;
  last.out_stride = n_targets;
  last.out_col = 0;
  last.y_in = yt;
  last.ld_out = logdens;
  rc = run_layers(m, st, rows, tps, kv, b, /*need_merge=*/n_buf > 0, last, s);
  if (rc) return rc;
  st->buffer_len = n_buf;
  return ARTAB_OK;
}

int artab_context_attention(int dtype, const void* q, const void* k_ctx, const void* v_ctx, int rows,
                            int rows_per_group, int n_groups, int n_heads, int head_dim, int n_ctx, int n_ctx_pad,
                            int n_splits, float* out, float* lse, int32_t* status, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(q && k_ctx && v_ctx && out && lse, ARTAB_EINVAL, "context_attention: null pointer");
  ARTAB_REQUIRE(rows >= 0 && n_groups >= 1 && n_heads >= 1 && n_ctx >= 1 && n_splits >= 1 && n_ctx_pad >= n_ctx,
                ARTAB_EINVAL, "context_attention: bad sizes");
  ARTAB_REQUIRE(n_groups == 1 || rows == rows_per_group * n_groups, ARTAB_EINVAL,
                "context_attention: rows must equal rows_per_group * n_groups");
  CtxAttnArgs c;
  memset(&c, 0, sizeof(c));
  c.dtype = dtype;
  c.q = q;
  c.k_ctx = k_ctx;
  c.v_ctx = v_ctx;
  c.v_transposed = dtype == ARTAB_BF16;
  c.rows = rows;
  c.rows_per_group = rows_per_group;
  c.n_groups = n_groups;
  c.n_heads = n_heads;
  c.head_dim = head_dim;
  c.n_ctx = n_ctx;
  c.n_ctx_pad = n_ctx_pad;
  c.n_splits = n_splits;
  c.scale = 1.0f / sqrtf((float)head_dim);
  c.out = out;
  c.lse = lse;
  c.status = status;
  return use_tc(dtype, head_dim) ? launch_ctx_attn_tc(c, (cudaStream_t)stream)
                                 : launch_ctx_attn_simt(c, (cudaStream_t)stream);
}

int artab_buffer_attention_merge(int dtype, const void* q, const void* kv_buf, int n_streams, int n_heads,
                                 int head_dim, int max_buf, int mode_tf, int n_new_or_nt, int len0,
                                 const float* o_part, const float* lse_part, int n_splits, int rows, float* out,
                                 void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(q && o_part && lse_part && out && n_splits >= 1, ARTAB_EINVAL, "buffer_attention_merge: null pointer");
  ARTAB_REQUIRE(kv_buf || (!mode_tf && len0 == 0), ARTAB_EINVAL, "buffer_attention_merge: kv_buf is null");
  ARTAB_REQUIRE(mode_tf ? (n_new_or_nt >= 1 && n_new_or_nt <= max_buf && rows == n_streams * 2 * n_new_or_nt)
                        : ((n_new_or_nt == 1 || n_new_or_nt == 2) && len0 >= 0 && len0 <= max_buf &&
                           rows == n_streams * n_new_or_nt),
                ARTAB_EINVAL, "buffer_attention_merge: inconsistent sizes");
  BufMergeArgs b;
  memset(&b, 0, sizeof(b));
  b.dtype = dtype;
  b.q = q;
  b.kv_buf = kv_buf;
  b.n_heads = n_heads;
  b.head_dim = head_dim;
  b.max_buf = max_buf;
  b.mode_tf = mode_tf;
  b.nt = mode_tf ? n_new_or_nt : 0;
  b.n_new = mode_tf ? 0 : n_new_or_nt;
  b.len0 = len0;
  b.n_items = mode_tf ? (long)n_streams * n_heads * (n_new_or_nt + 1) : (long)n_streams * n_heads;
  b.o_part = o_part;
  b.lse_part = lse_part;
  b.n_splits = n_splits;
  b.rows = rows;
  b.scale = 1.0f / sqrtf((float)head_dim);
  b.out = out;
  return launch_buf_merge(b, (cudaStream_t)stream);
}

int artab_buffer_attention_merge_ragged(int dtype, const void* q, const void* kv_buf, int n_streams, int n_heads,
                                        int head_dim, int max_buf, int n_new, const int32_t* lens, int len_max,
                                        const float* o_part, const float* lse_part, int n_splits, int rows,
                                        float* out, float* lse_out, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(q && o_part && lse_part && out && n_splits >= 1, ARTAB_EINVAL,
                "buffer_attention_merge_ragged: null pointer");
  ARTAB_REQUIRE(kv_buf || len_max == 0, ARTAB_EINVAL, "buffer_attention_merge_ragged: kv_buf is null");
  ARTAB_REQUIRE((n_new == 1 || n_new == 2) && len_max >= 0 && len_max <= max_buf && rows == n_streams * n_new,
                ARTAB_EINVAL, "buffer_attention_merge_ragged: inconsistent sizes");
  BufMergeArgs b;
  memset(&b, 0, sizeof(b));
  b.dtype = dtype;
  b.q = q;
  b.kv_buf = kv_buf;
  b.n_heads = n_heads;
  b.head_dim = head_dim;
  b.max_buf = max_buf;
  b.n_new = n_new;
  b.len0 = len_max;
  b.lens = lens;
  b.lse_out = lse_out;
  b.n_items = (long)n_streams * n_heads;
  b.o_part = o_part;
  b.lse_part = lse_part;
  b.n_splits = n_splits;
  b.rows = rows;
  b.scale = 1.0f / sqrtf((float)head_dim);
  b.out = out;
  return launch_buf_merge(b, (cudaStream_t)stream);
}

int artab_buffer_attention_merge_visible(int dtype, const void* q, const void* kv_buf, int n_streams, int n_heads,
                                         int head_dim, int max_buf, int tokens_per_stream, const int32_t* visible,
                                         int n_buf, const uint8_t* key_mask, const float* o_part,
                                         const float* lse_part, int n_splits, int rows, float* out, float* lse_out,
                                         void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(q && o_part && lse_part && out && visible && n_splits >= 1, ARTAB_EINVAL,
                "buffer_attention_merge_visible: null pointer");
  ARTAB_REQUIRE(kv_buf || n_buf == 0, ARTAB_EINVAL, "buffer_attention_merge_visible: kv_buf is null");
  ARTAB_REQUIRE(tokens_per_stream >= 1 && n_buf >= 0 && n_buf <= max_buf && rows == n_streams * tokens_per_stream,
                ARTAB_EINVAL, "buffer_attention_merge_visible: inconsistent sizes");
  BufMergeArgs b;
  memset(&b, 0, sizeof(b));
  b.dtype = dtype;
  b.q = q;
  b.kv_buf = kv_buf;
  b.n_heads = n_heads;
  b.head_dim = head_dim;
  b.max_buf = max_buf;
  b.mode_tf = 2;
  b.visible = visible;
  b.tps = tokens_per_stream;
  b.key_mask = key_mask;
  b.lse_out = lse_out;
  b.len0 = n_buf;  // upper bound of every visible count
  b.n_items = (long)n_streams * n_heads * tokens_per_stream;
  b.o_part = o_part;
  b.lse_part = lse_part;
  b.n_splits = n_splits;
  b.rows = rows;
  b.scale = 1.0f / sqrtf((float)head_dim);
  b.out = out;
  return launch_buf_merge(b, (cudaStream_t)stream);
}

int artab_kv_append(int dtype, void* kv_buf, const void* k_new, const void* v_new, int n_streams, int n_heads,
                    int head_dim, int max_buf, int pos, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(kv_buf && k_new && v_new, ARTAB_EINVAL, "kv_append: null pointer");
  ARTAB_REQUIRE(pos >= 0 && pos < max_buf, ARTAB_ECAPACITY,
                "Shared-context buffer cache exceeded; increase max buffer length.");
  return launch_kv_append(dtype, kv_buf, k_new, v_new, (long)n_streams * n_heads, head_dim, max_buf, pos,
                          (cudaStream_t)stream);
}

int artab_embed(const artab_model* m, const float* x, const float* y, const int32_t* ar_idx, int rows, int n_feat,
                int kind, float* out, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(m && x && out && n_feat > 0 && kind >= 0 && kind <= 2, ARTAB_EINVAL, "embed: bad argument");
  EmbedArgs e = embed_base(m);
  e.mode = EMB_ROWS;
  e.rows = rows;
  e.F = n_feat;
  e.kind = kind;
  e.x = x;
  e.y = y;
  e.ar_idx = ar_idx;
  e.out = out;
  return launch_embed(e, (cudaStream_t)stream);
}

static int head_common(const artab_model* m, const float* z, int rows, DenseArgs& d) {
  memset(&d, 0, sizeof(d));
  d.rows = rows;
  d.D = m->d_model;
  d.Dff = m->d_ff;
  d.n_comp = m->n_comp;
  d.x_in = z;
  d.do_head = 1;
  d.head_tps = 1;
  d.head_first = 0;
  d.out_stride = 1;
  d.out_col = 0;
  fill_head(m, d);
  return ARTAB_OK;
}

int artab_head_logpdf(const artab_model* m, const float* z, const float* y, int rows, float* logdens, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(m && z && y && logdens, ARTAB_EINVAL, "head_logpdf: null pointer");
  DenseArgs d;
  head_common(m, z, rows, d);
  d.head_mode = 2;
  d.y_in = y;
  d.ld_out = logdens;
  return launch_dense(d, (cudaStream_t)stream);
}

int artab_head_sample(const artab_model* m, const float* z, const float* expo, const float* normal, int rows,
                      float* y, float* logdens, int32_t* comp, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(m && z && expo && normal && y, ARTAB_EINVAL, "head_sample: null pointer");
  DenseArgs d;
  head_common(m, z, rows, d);
  d.head_mode = 1;
  d.expo = expo;
  d.normal = normal;
  d.y_out = y;
  d.ld_out = logdens;
  d.comp_out = comp;
  return launch_dense(d, (cudaStream_t)stream);
}

}  // extern "C"
