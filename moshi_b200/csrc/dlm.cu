// Decoder-LM handle: a language model given as a list of layers (mixer + feed-forward per layer), its weights under the
// checkpoint's names, a slot cache of per-layer latents, and the ragged step (any number of new tokens per slot) that both
// prompt portions and single-token decoding go through.  The Likosun design is the first user of the registered mechanisms.
#include <algorithm>

#include "dlm_kernels.cuh"
#include "gemm_sk.cuh"
#include "lm_kernels.cuh"

using namespace b200;
using namespace b200::dlm;

namespace {

// a linear's weight: row-major [N][K] of the compute type, or (bf16, eligible shape) the packed tiles of the tcgen05 GEMM
struct Weight {
  void* rm = nullptr;
  void* tiles = nullptr;
  int N = 0, K = 0;
};

struct Layer {
  b200_dlm_layer c;
  int ncat = 0, ldp = 0, off_q = 0, off_dkv = 0, off_up = 0, off_g1 = 0, off_g2 = 0;
  Weight cat, o, down;                 // [q | dkv | up | gate1 | gate2] x width;  width x (heads * vdim);  width x ff
  void *ukT = nullptr, *uv = nullptr;  // [H][r][dim] (transposed per head), [H * vdim][r]
  float *n1w = nullptr, *n1b = nullptr, *cnorm = nullptr, *sink = nullptr, *b1 = nullptr, *b2 = nullptr, *avg = nullptr;
  void* cache = nullptr;               // [slots][cap][r]
  int sig = 0;                         // index of the layer's attention tile list
};

// attention tile list of one (heads, rows per tile) combination
struct TileSig {
  int H, rpt;
  int off_row0 = 0, off_rows = 0, off_slot = 0;     // offsets into the step's metadata block (ints)
  int count = 0;
};

}  // namespace

struct b200_dlm {
  b200_dlm_config cfg;
  std::vector<Layer> layers;
  TensorStore store;
  Arena weights, state;
  bool finalized = false, f32 = false;
  int device = -1;
  int use_tc = 1, trace_layers = 0, attn_split = 0, attn_tc = 1;
  // option "time_kernels": CUDA events around every operation of a step, summed per class (bench.py's per-kernel roofline)
  int time_kernels = 0;
  std::vector<cudaEvent_t> ev_pool; std::vector<int> ev_class; size_t ev_used = 0;
  double class_ms[4] = {0, 0, 0, 0};
  void *embed = nullptr;
  Weight head;
  float *fnw = nullptr, *fnb = nullptr;
  int64_t weight_bytes = 0;
  // cache and step buffers
  int slots = 0, cap = 0, tmax = 0, wmax = 0;
  std::vector<int> len;                // tokens held per slot
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_meta = nullptr;
  int *meta_dev = nullptr, *meta_pin = nullptr; int meta_ints = 0;
  int off_tok = 0, off_slot = 0, off_pos = 0, off_want = 0;
  std::vector<TileSig> sigs;
  float *xin = nullptr, *stack = nullptr, *trace = nullptr, *qa = nullptr, *ol = nullptr, *part = nullptr, *logits = nullptr;
  void *hbuf = nullptr, *proj = nullptr, *obuf = nullptr, *mixo = nullptr, *act = nullptr, *ffo = nullptr, *hf = nullptr;
  bf16 *logits_bf = nullptr, *head_bf = nullptr;
  size_t part_floats = 0;
  int last_tokens = 0, last_want = 0;
  int* err = nullptr;
  float* sk_ws = nullptr; int* sk_counters = nullptr;
  tc::GemmPlanCache plans;
};

namespace {

size_t esize(const b200_dlm* h) { return h->f32 ? 4 : 2; }
int rows_per_tile(int r) { return r <= 512 ? 16 : 8; }

template <typename TO>
int convert_into(const Tensor* t, TO* dst) {
  const long long n = t->numel();
  const unsigned g = (unsigned)ceil_div64(n, 256);
  if (t->dtype == B200_BF16) B200_LAUNCH(convert_kernel, g, 256, 0, nullptr, static_cast<const bf16*>(t->data), dst, n);
  else if (t->dtype == B200_F32) B200_LAUNCH(convert_kernel, g, 256, 0, nullptr, static_cast<const float*>(t->data), dst, n);
  else B200_FAIL(B200_ERR_SHAPE, "decoder LM: weights must be bfloat16 or float32");
  return check_launch("convert");
}

int find_tensor(b200_dlm* h, const std::string& name, std::vector<int64_t> shape, const Tensor** out) {
  const Tensor* t = h->store.find(name);
  if (!t) B200_FAIL(B200_ERR_MISSING, "decoder LM finalize: tensor '%s' was not loaded", name.c_str());
  if (t->shape != shape) {
    std::string got;
    for (auto s : t->shape) got += std::to_string(s) + ",";
    B200_FAIL(B200_ERR_SHAPE, "decoder LM tensor '%s' has shape [%s]", name.c_str(), got.c_str());
  }
  *out = t;
  return B200_OK;
}

// small vectors always live in fp32
int get_f32(b200_dlm* h, const std::string& name, int64_t n, float** out) {
  const Tensor* t = nullptr;
  B200_TRY(find_tensor(h, name, {n}, &t));
  B200_TRY(h->weights.alloc_t(out, (size_t)n, false));
  h->weight_bytes += n * 4;
  return convert_into(t, *out);
}

// matrix rows [rows][K] of the compute type written at dst (row offset inside a concatenation)
int put_matrix(b200_dlm* h, const std::string& name, int64_t rows, int64_t K, void* dst) {
  const Tensor* t = nullptr;
  B200_TRY(find_tensor(h, name, {rows, K}, &t));
  return h->f32 ? convert_into(t, static_cast<float*>(dst)) : convert_into(t, static_cast<bf16*>(dst));
}

// bf16 mode + eligible shape: the row-major matrix is replaced by the tcgen05 GEMM's packed tiles
int seal_weight(b200_dlm* h, Weight& w, void* rm, int N, int K, std::vector<void*>& drop) {
  w.rm = rm; w.N = N; w.K = K; w.tiles = nullptr;
  h->weight_bytes += (int64_t)N * K * esize(h);
  if (!h->f32 && h->use_tc && K >= 8 && K % 8 == 0 && (N + 127) / 128 <= tc::SK_MAX_TILES) {
    B200_TRY(h->weights.alloc(&w.tiles, tc::sk_packed_bytes(N, K, 0, 0), false));
    B200_TRY(tc::sk_pack_weights(static_cast<const bf16*>(rm), w.tiles, N, K, 0, 0, nullptr));
    drop.push_back(rm);
    w.rm = nullptr;
  }
  return B200_OK;
}

template <typename TA, typename TB, typename TC>
int gemm_nt(cudaStream_t st, const TA* A, long long lda, long long sa, const TB* B, long long ldb, long long sb, TC* C, long long ldc,
            long long sc, int M, int N, int K, int batch, float alpha) {
  dim3 grid(ceil_div(N, 64), ceil_div(M, 64), batch);
  B200_LAUNCH((gemm_nt_kernel<TA, TB, TC>), grid, 256, 0, st, A, lda, sa, B, ldb, sb, C, ldc, sc, M, N, K, alpha);
  return check_launch("gemm_nt");
}

// the per-head products around the latent attention: tensor cores for bf16 weights (K a multiple of 16), else CUDA cores
template <typename TA, typename TB, typename TC>
int head_gemm(cudaStream_t st, const TA* A, long long lda, long long sa, const TB* B, long long ldb, long long sb, TC* C, long long ldc,
              long long sc, int M, int N, int K, int batch, float alpha, bool tensor_cores) {
  if constexpr (sizeof(TB) == 2) {
    constexpr long long AE = 16 / (long long)sizeof(TA);       // elements of A per 16 bytes
    const bool aligned = lda % AE == 0 && sa % AE == 0 && ldb % 8 == 0 && sb % 8 == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)B % 16 == 0;
    if (tensor_cores && K % 16 == 0 && aligned) {
      dim3 grid(ceil_div(N, 64), ceil_div(M, 64), batch);
      B200_LAUNCH((gemm_nt_mma_kernel<TA, TC>), grid, 128, 0, st, A, lda, sa, B, ldb, sb, C, ldc, sc, M, N, K, alpha);
      return check_launch("gemm_nt_mma");
    }
  }
  return gemm_nt(st, A, lda, sa, B, ldb, sb, C, ldc, sc, M, N, K, batch, alpha);
}

// y[M][N] = x[M][K] . W^T in the compute type
template <typename T>
int linear(b200_dlm* h, const T* x, long long ldx, const Weight& w, T* y, long long ldy, int M);

template <>
int linear<float>(b200_dlm* h, const float* x, long long ldx, const Weight& w, float* y, long long ldy, int M) {
  return gemm_nt(h->stream, x, ldx, 0, static_cast<const float*>(w.rm), (long long)w.K, 0, y, ldy, 0, M, w.N, w.K, 1, 1.f);
}

template <>
int linear<bf16>(b200_dlm* h, const bf16* x, long long ldx, const Weight& w, bf16* y, long long ldy, int M) {
  if (w.tiles && ldx % 8 == 0 && ldy % 8 == 0) {
    tc::SkTuning t;
    for (int m0 = 0; m0 < M; m0 += 256) {          // the LM's GEMM takes up to 256 rows per launch
      const int m = std::min(256, M - m0);
      B200_TRY(tc::sk_linear(h->plans, x + (long long)m0 * ldx, ldx, w.tiles, y + (long long)m0 * ldy, ldy, nullptr, 0, m, w.N, w.K, 0, 0,
                             h->sk_ws, h->sk_counters, t, h->stream));
    }
    return B200_OK;
  }
  if (!w.rm) B200_FAIL(B200_ERR_STATE, "decoder LM: a packed linear met an unaligned activation stride");
  return gemm_nt(h->stream, x, ldx, 0, static_cast<const bf16*>(w.rm), (long long)w.K, 0, y, ldy, 0, M, w.N, w.K, 1, 1.f);
}

template <typename T, int NCH, int RPW>
int launch_attn(cudaStream_t st, const AttnParams& p, int tiles, int nsplit) {
  const size_t smem = (size_t)32 * p.r * sizeof(T);
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    B200_CUDA(cudaFuncSetAttribute(latent_attn_kernel<T, NCH, RPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set = true;
  }
  B200_LAUNCH((latent_attn_kernel<T, NCH, RPW>), dim3(tiles, nsplit), 128, smem, st, p);
  return check_launch("latent_attn");
}

// keys are cut over `nsplit` CTAs per tile when the tiles alone cannot fill the GPU (decoding, short portions)
int pick_split(int forced, int tiles, int max_ctx, int rpt, int r, size_t part_floats) {
  const int key_tiles = ceil_div(max_ctx, 32);
  int nsplit = 1;
  if (forced > 0) nsplit = std::min(forced, 64);
  else if (tiles < 148) nsplit = std::min(std::max(444 / tiles, 1), 64);      // one wave of three CTAs per SM
  nsplit = std::max(1, std::min(nsplit, key_tiles));
  nsplit = ceil_div(key_tiles, ceil_div(key_tiles, nsplit));                   // no split without a key tile
  while (nsplit > 1 && (size_t)tiles * nsplit * rpt * (r + 2) > part_floats) --nsplit;
  return nsplit;
}

template <int NKS>
int launch_attn_mma(cudaStream_t st, const AttnParams& p, int tiles) {
  const size_t smem = (size_t)2 * 32 * (p.r + 8) * 2 + (size_t)4 * 16 * 32 * 4 + (size_t)16 * 40 * 2 + (size_t)3 * 16 * 4 + 16;      // keys, partial scores, weights, row state, mbarriers
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(latent_attn_mma_kernel<NKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    attr_set = true;
  }
  B200_LAUNCH(latent_attn_mma_kernel<NKS>, dim3(tiles, p.nsplit), 128, smem, st, p);
  return check_launch("latent_attn_mma");
}

// bf16 latents of 64, 128, .., 512 elements take the tensor-core kernel
inline bool attn_mma_takes(int r, int rpt, bool bf16_latents) { return bf16_latents && rpt == 16 && r % 64 == 0 && r <= 512; }

template <typename T>
int run_attention(cudaStream_t st, AttnParams p, int tiles, int rpt, bool tensor_cores = true) {
  const int r = p.r;
  if (tensor_cores && attn_mma_takes(r, rpt, sizeof(T) == 2)) {
    switch (r / 64) {
      case 1: B200_TRY(launch_attn_mma<1>(st, p, tiles)); break;
      case 2: B200_TRY(launch_attn_mma<2>(st, p, tiles)); break;
      case 3: B200_TRY(launch_attn_mma<3>(st, p, tiles)); break;
      case 4: B200_TRY(launch_attn_mma<4>(st, p, tiles)); break;
      case 5: B200_TRY(launch_attn_mma<5>(st, p, tiles)); break;
      case 6: B200_TRY(launch_attn_mma<6>(st, p, tiles)); break;
      case 7: B200_TRY(launch_attn_mma<7>(st, p, tiles)); break;
      default: B200_TRY(launch_attn_mma<8>(st, p, tiles)); break;
    }
  }
  else if (r <= 64) B200_TRY((launch_attn<T, 2, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 128) B200_TRY((launch_attn<T, 4, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 256) B200_TRY((launch_attn<T, 8, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 512) B200_TRY((launch_attn<T, 16, 4>(st, p, tiles, p.nsplit)));
  else B200_TRY((launch_attn<T, 32, 2>(st, p, tiles, p.nsplit)));
  if (p.nsplit > 1) {
    B200_LAUNCH(latent_attn_merge_kernel, dim3(tiles, rpt), 128, 0, st, p.part, p.tile_row0, p.tile_rows, p.out, r, p.nsplit, rpt);
    B200_TRY(check_launch("latent_attn_merge"));
  }
  return B200_OK;
}

template <typename T>
int attention(b200_dlm* h, const Layer& L, int max_ctx) {
  const TileSig& s = h->sigs[L.sig];
  AttnParams p;
  p.qa = h->qa; p.cache = L.cache; p.sink = L.sink;
  p.tile_row0 = h->meta_dev + s.off_row0; p.tile_rows = h->meta_dev + s.off_rows; p.tile_slot = h->meta_dev + s.off_slot;
  p.tok_pos = h->meta_dev + h->off_pos;
  p.out = h->ol; p.part = h->part; p.cap = h->cap; p.r = L.c.kv_rank; p.H = L.c.heads; p.err = h->err;
  p.nsplit = pick_split(h->attn_split, s.count, max_ctx, s.rpt, p.r, h->part_floats);
  return run_attention<T>(h->stream, p, s.count, s.rpt, h->attn_tc != 0);
}

enum { CLS_LINEAR = 0, CLS_ATTN = 1, CLS_FOLD = 2, CLS_ELEMENTWISE = 3 };

int mark(b200_dlm* h, int cls) {       // cls >= 0 opens an interval of that class, -1 closes the open one
  if (!h->time_kernels) return B200_OK;
  if (h->ev_used == h->ev_pool.size()) {
    cudaEvent_t e;
    B200_CUDA(cudaEventCreate(&e));
    h->ev_pool.push_back(e); h->ev_class.push_back(0);
  }
  h->ev_class[h->ev_used] = cls;
  B200_CUDA(cudaEventRecord(h->ev_pool[h->ev_used++], h->stream));
  return B200_OK;
}
#define TIMED(cls, ...) do { B200_TRY(mark(h, cls)); __VA_ARGS__; B200_TRY(mark(h, -1)); } while (0)

template <typename T>
int step_body(b200_dlm* h, int n_tok, int n_want, int max_ctx, float* logits_out) {
  const b200_dlm_config& c = h->cfg;
  const int W = c.width;
  cudaStream_t st = h->stream;
  const int* meta = h->meta_dev;
  const long long stride = (long long)h->tmax * W;
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(embed_kernel<T>, n_tok, 256, 0, st, meta + h->off_tok, static_cast<const T*>(h->embed), c.vocab, W, c.embedding_scale,
              h->xin, h->stack, h->err));
  T* hb = static_cast<T*>(h->hbuf);
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(layernorm_kernel<T>, n_tok, 256, 0, st, h->xin, (const int*)nullptr, h->layers[0].n1w, h->layers[0].n1b, hb, W, c.norm_eps));
  for (int li = 0; li < c.n_layers; ++li) {
    const Layer& L = h->layers[li];
    const int H = L.c.heads, dk = L.c.dim, dv = L.c.vdim, r = L.c.kv_rank;
    T* proj = static_cast<T*>(h->proj);
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, hb, W, L.cat, proj, L.ldp, n_tok)));
    // mixer: latent attention
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(latent_append_kernel<T>, ceil_div(n_tok, 4), 128, 0, st, proj, (long long)L.ldp, L.off_dkv, L.cnorm, static_cast<T*>(L.cache),
                h->cap, r, meta + h->off_slot, meta + h->off_pos, n_tok, c.norm_eps));
    // query folded through W_uk (and the score scale): qa[t][h][:] = scale * q[t][h][:] . W_uk[h]
    TIMED(CLS_FOLD, B200_TRY(head_gemm(st, proj + L.off_q, (long long)L.ldp, (long long)dk, static_cast<const T*>(L.ukT), (long long)dk, (long long)r * dk, h->qa,
                     (long long)H * r, (long long)r, n_tok, r, dk, H, L.c.scale, h->attn_tc != 0)));
    TIMED(CLS_ATTN, B200_TRY(attention<T>(h, L, max_ctx)));
    // values: o[t][h][:] = W_uv[h] . (sum_j p_j c_j)
    T* ob = static_cast<T*>(h->obuf);
    TIMED(CLS_FOLD, B200_TRY(head_gemm(st, h->ol, (long long)H * r, (long long)r, static_cast<const T*>(L.uv), (long long)r, (long long)dv * r, ob, (long long)H * dv,
                     (long long)dv, n_tok, dv, r, H, 1.f, h->attn_tc != 0)));
    T* mixo = static_cast<T*>(h->mixo);
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)H * dv, L.o, mixo, W, n_tok)));
    // feed-forward
    T* ffo = nullptr;
    if (L.c.mlp == B200_MLP_DENSE_RELU2) {
      T* act = static_cast<T*>(h->act);
      const long long n = (long long)n_tok * L.c.ff;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(relu2_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, st, proj, (long long)L.ldp, L.off_up, act, L.c.ff, n));
      ffo = static_cast<T*>(h->ffo);
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, act, L.c.ff, L.down, ffo, W, n_tok)));
    }
    const bool last = li + 1 == c.n_layers;
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(block_end_kernel<T>, n_tok, 256, 0, st, h->xin, mixo, ffo, proj, (long long)L.ldp, L.off_g1, L.off_g2, L.b1, L.b2, c.residual_mult,
                h->stack, stride, li, L.avg, h->trace_layers ? h->trace + (long long)li * stride : nullptr,
                last ? nullptr : h->layers[li + 1].n1w, last ? nullptr : h->layers[li + 1].n1b, hb, W, c.norm_eps));
  }
  B200_TRY(check_launch("decoder LM layers"));
  if (n_want > 0) {
    T* hf = static_cast<T*>(h->hf);
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(layernorm_kernel<T>, n_want, 256, 0, st, h->xin, meta + h->off_want, h->fnw, h->fnb, hf, W, c.norm_eps));
    if (h->head.tiles) {
      const int ldl = (c.vocab + 7) / 8 * 8;
      TIMED(CLS_LINEAR, B200_TRY(linear<bf16>(h, reinterpret_cast<const bf16*>(hf), W, h->head, h->head_bf, ldl, n_want)));
      const long long n = (long long)n_want * c.vocab;
      B200_LAUNCH(rows_to_f32_kernel, (unsigned)ceil_div64(n, 256), 256, 0, st, h->head_bf, (long long)ldl, h->logits, c.vocab, n);
    } else {
      TIMED(CLS_LINEAR, B200_TRY(gemm_nt(st, hf, (long long)W, 0, static_cast<const T*>(h->head.rm), (long long)W, 0, h->logits, (long long)c.vocab, 0, n_want, c.vocab, W, 1, 1.f)));
    }
    if (logits_out)
      B200_CUDA(cudaMemcpyAsync(logits_out, h->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToDevice, st));
  }
  return check_launch("decoder LM step");
}

}  // namespace

extern "C" {

int b200_dlm_create(const b200_dlm_config* cfg, b200_dlm** out) {
  if (!cfg || !out || !cfg->layers) B200_FAIL(B200_ERR_INVALID, "dlm_create: null argument");
  if (cfg->vocab < 1 || cfg->width < 1 || cfg->n_layers < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: vocab, width and n_layers must be positive");
  if (cfg->compute_dtype != B200_BF16 && cfg->compute_dtype != B200_F32) B200_FAIL(B200_ERR_INVALID, "dlm_create: compute_dtype must be bf16 or f32");
  for (int i = 0; i < cfg->n_layers; ++i) {
    const b200_dlm_layer& l = cfg->layers[i];
    if (l.mixer != B200_MIXER_LATENT_ATTENTION) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: unknown mixer %d", i, l.mixer);
    if (l.heads < 1 || l.dim < 1 || l.vdim < 1 || l.kv_rank < 1 || l.kv_rank > 1024)
      B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: heads, dim, vdim must be positive and kv_rank in 1..1024", i);
    if (l.mlp != B200_MLP_NONE && l.mlp != B200_MLP_DENSE_RELU2) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: unknown mlp kind %d", i, l.mlp);
    if (l.mlp != B200_MLP_NONE && l.ff < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: ff must be positive", i);
  }
  auto* h = new b200_dlm();
  h->cfg = *cfg;
  h->layers.resize(cfg->n_layers);
  for (int i = 0; i < cfg->n_layers; ++i) h->layers[i].c = cfg->layers[i];
  h->cfg.layers = nullptr;
  h->f32 = cfg->compute_dtype == B200_F32;
  if (cudaGetDevice(&h->device) != cudaSuccess) h->device = -1;
  *out = h;
  return B200_OK;
}

int b200_dlm_load_tensor(b200_dlm* h, const char* name, const void* data_dev, int dtype, int ndim, const int64_t* shape) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_load_tensor: null handle");
  if (h->finalized) B200_FAIL(B200_ERR_STATE, "dlm_load_tensor: the model is finalized");
  DeviceGuard g(h->device);
  return h->store.put(name, data_dev, dtype, ndim, shape);
}

int b200_dlm_set_option(b200_dlm* h, const char* name, int value) {
  if (!h || !name) B200_FAIL(B200_ERR_INVALID, "dlm_set_option: null argument");
  const std::string n(name);
  if (n == "use_tc") {
    if (h->finalized) B200_FAIL(B200_ERR_STATE, "dlm_set_option: use_tc is fixed once the weights are packed");
    h->use_tc = value != 0;
  } else if (n == "trace_layers") {
    if (h->slots) B200_FAIL(B200_ERR_STATE, "dlm_set_option: trace_layers must be set before cache_begin");
    h->trace_layers = value != 0;
  } else if (n == "attn_tc") {
    h->attn_tc = value != 0;
  } else if (n == "time_kernels") {
    h->time_kernels = value != 0;
  } else if (n == "attn_split") {
    h->attn_split = value < 0 ? 0 : value;
  } else {
    B200_FAIL(B200_ERR_INVALID, "dlm_set_option: unknown option '%s'", name);
  }
  return B200_OK;
}

int b200_dlm_finalize(b200_dlm* h) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_finalize: null handle");
  if (h->finalized) return B200_OK;
  DeviceGuard g(h->device);
  const b200_dlm_config& c = h->cfg;
  const int64_t W = c.width;
  const size_t es = esize(h);
  std::vector<void*> drop;
  auto matrix = [&](const std::string& name, int64_t rows, int64_t K, void** out) -> int {
    B200_TRY(h->weights.alloc(out, (size_t)rows * K * es, false));
    return put_matrix(h, name, rows, K, *out);
  };
  B200_TRY(matrix("embed", c.vocab, W, &h->embed));
  h->weight_bytes += (int64_t)c.vocab * W * es;
  for (int i = 0; i < c.n_layers; ++i) {
    Layer& L = h->layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const int64_t H = L.c.heads, dk = L.c.dim, dv = L.c.vdim, r = L.c.kv_rank, F = L.c.ff;
    const bool mlp = L.c.mlp != B200_MLP_NONE;
    B200_TRY(get_f32(h, p + "norm1", W, &L.n1w));
    B200_TRY(get_f32(h, p + "norm1.b", W, &L.n1b));
    // one matrix for everything that reads the normed input: q | latent | up | gate of the mixer | gate of the feed-forward
    L.off_q = 0; L.off_dkv = (int)(H * dk); L.off_up = L.off_dkv + (int)r; L.off_g1 = L.off_up + (mlp ? (int)F : 0);
    L.off_g2 = L.off_g1 + (int)W; L.ncat = L.off_g2 + (mlp ? (int)W : 0);
    L.ldp = (L.ncat + 7) / 8 * 8;
    void* cat = nullptr;
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, false));
    auto at = [&](int off) { return static_cast<char*>(cat) + (size_t)off * W * es; };
    B200_TRY(put_matrix(h, p + "mix.q", H * dk, W, at(L.off_q)));
    B200_TRY(put_matrix(h, p + "mix.dkv", r, W, at(L.off_dkv)));
    if (mlp) B200_TRY(put_matrix(h, p + "mlp.up", F, W, at(L.off_up)));
    B200_TRY(put_matrix(h, p + "rg1", W, W, at(L.off_g1)));
    if (mlp) B200_TRY(put_matrix(h, p + "rg2", W, W, at(L.off_g2)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    B200_TRY(get_f32(h, p + "rg1.b", W, &L.b1));
    if (mlp) B200_TRY(get_f32(h, p + "rg2.b", W, &L.b2));
    B200_TRY(get_f32(h, p + "mix.dkv.norm", r, &L.cnorm));
    B200_TRY(get_f32(h, p + "mix.sink", H, &L.sink));
    {   // W_uk [H * dim][r] -> per head [r][dim]
      void* uk = nullptr;
      B200_TRY(matrix(p + "mix.uk", H * dk, r, &uk));
      B200_TRY(h->weights.alloc(&L.ukT, (size_t)H * dk * r * es, false));
      const long long n = H * dk * r;
      if (h->f32) B200_LAUNCH(head_transpose_kernel<float>, (unsigned)ceil_div64(n, 256), 256, 0, nullptr, static_cast<const float*>(uk), static_cast<float*>(L.ukT), (int)H, (int)dk, (int)r);
      else B200_LAUNCH(head_transpose_kernel<bf16>, (unsigned)ceil_div64(n, 256), 256, 0, nullptr, static_cast<const bf16*>(uk), static_cast<bf16*>(L.ukT), (int)H, (int)dk, (int)r);
      B200_TRY(check_launch("head_transpose"));
      drop.push_back(uk);
      h->weight_bytes += n * es;
    }
    B200_TRY(matrix(p + "mix.uv", H * dv, r, &L.uv));
    h->weight_bytes += H * dv * r * es;
    void* wo = nullptr;
    B200_TRY(matrix(p + "mix.o", W, H * dv, &wo));
    B200_TRY(seal_weight(h, L.o, wo, (int)W, (int)(H * dv), drop));
    if (mlp) {
      void* wd = nullptr;
      B200_TRY(matrix(p + "mlp.down", W, F, &wd));
      B200_TRY(seal_weight(h, L.down, wd, (int)W, (int)F, drop));
    }
    B200_TRY(get_f32(h, p + "dwa", i + 2, &L.avg));
    int sig = -1;
    const int rpt = rows_per_tile((int)r);
    for (size_t k = 0; k < h->sigs.size(); ++k) if (h->sigs[k].H == H && h->sigs[k].rpt == rpt) sig = (int)k;
    if (sig < 0) { TileSig s; s.H = (int)H; s.rpt = rpt; h->sigs.push_back(s); sig = (int)h->sigs.size() - 1; }
    L.sig = sig;
  }
  B200_TRY(get_f32(h, "final.norm", W, &h->fnw));
  B200_TRY(get_f32(h, "final.norm.b", W, &h->fnb));
  void* hd = nullptr;
  B200_TRY(matrix("head", c.vocab, W, &hd));
  B200_TRY(seal_weight(h, h->head, hd, c.vocab, (int)W, drop));
  B200_CUDA(cudaDeviceSynchronize());
  for (void* p : drop) {
    auto it = std::find(h->weights.ptrs.begin(), h->weights.ptrs.end(), p);
    if (it != h->weights.ptrs.end()) h->weights.ptrs.erase(it);
    cudaFree(p);
  }
  h->store.release_all();
  h->finalized = true;
  return B200_OK;
}

int b200_dlm_cache_end(b200_dlm* h) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_cache_end: null handle");
  DeviceGuard g(h->device);
  if (h->slots) cudaStreamSynchronize(h->stream);
  h->state.free_all();
  if (h->meta_pin) { cudaFreeHost(h->meta_pin); h->meta_pin = nullptr; }
  for (auto e : h->ev_pool) cudaEventDestroy(e);
  h->ev_pool.clear(); h->ev_class.clear(); h->ev_used = 0;
  if (h->ev_meta) { cudaEventDestroy(h->ev_meta); h->ev_meta = nullptr; }
  h->plans.clear();
  h->slots = h->cap = h->tmax = h->wmax = 0;
  h->len.clear();
  return B200_OK;
}

int b200_dlm_destroy(b200_dlm* h) {
  if (!h) return B200_OK;
  b200_dlm_cache_end(h);
  DeviceGuard g(h->device);
  h->weights.free_all();
  h->store.release_all();
  delete h;
  return B200_OK;
}

int b200_dlm_set_stream(b200_dlm* h, void* stream) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_set_stream: null handle");
  h->stream = static_cast<cudaStream_t>(stream);
  return B200_OK;
}

int b200_dlm_cache_begin(b200_dlm* h, int slots, int capacity, int max_step_tokens, int max_want, void* stream) {
  if (!h || !h->finalized) B200_FAIL(B200_ERR_STATE, "dlm_cache_begin: finalize the model first");
  if (h->slots) B200_FAIL(B200_ERR_STATE, "dlm_cache_begin: the cache exists already");
  if (slots < 1 || capacity < 1 || max_step_tokens < 1 || max_want < 1) B200_FAIL(B200_ERR_INVALID, "dlm_cache_begin: sizes must be positive");
  DeviceGuard g(h->device);
  const b200_dlm_config& c = h->cfg;
  Arena& A = h->state;
  const size_t es = esize(h);
  const size_t T = (size_t)max_step_tokens, W = (size_t)c.width;
  h->stream = static_cast<cudaStream_t>(stream);
  size_t max_ldp = 0, max_hr = 0, max_hv = 0, max_ff = 1, max_r = 0, max_tiles = 0;
  for (auto& L : h->layers) {
    B200_TRY(A.alloc(&L.cache, (size_t)slots * capacity * L.c.kv_rank * es));
    max_ldp = std::max(max_ldp, (size_t)L.ldp);
    max_hr = std::max(max_hr, (size_t)L.c.heads * L.c.kv_rank);
    max_hv = std::max(max_hv, (size_t)L.c.heads * L.c.vdim);
    max_ff = std::max(max_ff, (size_t)L.c.ff);
    max_r = std::max(max_r, (size_t)L.c.kv_rank);
  }
  B200_TRY(A.alloc_t(&h->xin, T * W));
  B200_TRY(A.alloc_t(&h->stack, (size_t)(c.n_layers + 1) * T * W));
  if (h->trace_layers) B200_TRY(A.alloc_t(&h->trace, (size_t)c.n_layers * T * W));
  B200_TRY(A.alloc_t(&h->qa, T * max_hr));
  B200_TRY(A.alloc_t(&h->ol, T * max_hr));
  h->part_floats = (size_t)600 * 16 * (max_r + 2);
  B200_TRY(A.alloc_t(&h->part, h->part_floats));
  B200_TRY(A.alloc(&h->hbuf, T * W * es));
  B200_TRY(A.alloc(&h->proj, T * max_ldp * es));
  B200_TRY(A.alloc(&h->obuf, T * max_hv * es));
  B200_TRY(A.alloc(&h->mixo, T * W * es));
  B200_TRY(A.alloc(&h->act, T * max_ff * es));
  B200_TRY(A.alloc(&h->ffo, T * W * es));
  B200_TRY(A.alloc(&h->hf, (size_t)max_want * W * es));
  B200_TRY(A.alloc_t(&h->logits, (size_t)max_want * c.vocab));
  B200_TRY(A.alloc_t(&h->logits_bf, (size_t)max_want * c.vocab));
  B200_TRY(A.alloc_t(&h->head_bf, (size_t)max_want * ((c.vocab + 7) / 8 * 8)));
  B200_TRY(A.alloc_t(&h->err, 1));
  B200_TRY(A.alloc(reinterpret_cast<void**>(&h->sk_ws), tc::sk_workspace_bytes(256), false));
  B200_TRY(A.alloc_t(&h->sk_counters, tc::SK_MAX_TILES));
  // step metadata: tokens | slot | position per token, wanted rows, then one tile list per (heads, rows per tile) combination
  int off = 0;
  h->off_tok = off; off += max_step_tokens;
  h->off_slot = off; off += max_step_tokens;
  h->off_pos = off; off += max_step_tokens;
  h->off_want = off; off += max_want;
  for (auto& s : h->sigs) {
    max_tiles = (size_t)ceil_div64((int64_t)max_step_tokens * s.H, s.rpt) + (size_t)std::min(slots, max_step_tokens);
    s.off_row0 = off; off += (int)max_tiles;
    s.off_rows = off; off += (int)max_tiles;
    s.off_slot = off; off += (int)max_tiles;
  }
  h->meta_ints = off;
  B200_TRY(A.alloc_t(&h->meta_dev, (size_t)off));
  B200_CUDA(cudaMallocHost(&h->meta_pin, (size_t)off * sizeof(int)));
  B200_CUDA(cudaEventCreateWithFlags(&h->ev_meta, cudaEventDisableTiming));
  h->slots = slots; h->cap = capacity; h->tmax = max_step_tokens; h->wmax = max_want;
  h->len.assign(slots, 0);
  h->last_tokens = h->last_want = 0;
  if (!h->f32 && h->use_tc) B200_TRY(tc::prepare_plans(h->plans));
  B200_CUDA(cudaDeviceSynchronize());
  return B200_OK;
}

int b200_dlm_release(b200_dlm* h, int slot) {
  if (!h || slot < 0 || slot >= h->slots) B200_FAIL(B200_ERR_INVALID, "dlm_release: slot %d does not exist", slot);
  h->len[slot] = 0;
  return B200_OK;
}

int b200_dlm_slot_length(b200_dlm* h, int slot) {
  if (!h || slot < 0 || slot >= h->slots) return -1;
  return h->len[slot];
}

int b200_dlm_step(b200_dlm* h, int n_entries, const int32_t* slots_host, const int32_t* counts_host, const int32_t* tokens_host,
                  int n_want, const int32_t* want_host, float* logits_dev) {
  if (!h || !h->slots) B200_FAIL(B200_ERR_STATE, "dlm_step: no cache (call cache_begin)");
  if (n_entries < 1 || !slots_host || !counts_host || !tokens_host || (n_want > 0 && !want_host)) B200_FAIL(B200_ERR_INVALID, "dlm_step: null argument");
  DeviceGuard g(h->device);
  long long total = 0;
  std::vector<char> used(h->slots, 0);
  for (int e = 0; e < n_entries; ++e) {
    const int s = slots_host[e], n = counts_host[e];
    if (s < 0 || s >= h->slots) B200_FAIL(B200_ERR_INVALID, "dlm_step: slot %d does not exist", s);
    if (used[s]) B200_FAIL(B200_ERR_INVALID, "dlm_step: slot %d appears twice in one step", s);
    used[s] = 1;
    if (n < 1) B200_FAIL(B200_ERR_INVALID, "dlm_step: entry %d brings no token", e);
    if (h->len[s] + n > h->cap) B200_FAIL(B200_ERR_STATE, "dlm_step: slot %d would hold %d tokens, capacity is %d", s, h->len[s] + n, h->cap);
    total += n;
  }
  if (total > h->tmax) B200_FAIL(B200_ERR_SHAPE, "dlm_step: %lld tokens in one step, the buffers take %d", total, h->tmax);
  if (n_want > h->wmax) B200_FAIL(B200_ERR_SHAPE, "dlm_step: %d logit rows wanted, the buffers take %d", n_want, h->wmax);
  for (int i = 0; i < n_want; ++i)
    if (want_host[i] < 0 || want_host[i] >= total) B200_FAIL(B200_ERR_INVALID, "dlm_step: wanted row %d is outside the step", want_host[i]);
  // the previous step's metadata copy must have left the pinned block
  B200_CUDA(cudaEventSynchronize(h->ev_meta));
  int* m = h->meta_pin;
  int t = 0, max_ctx = 0;
  for (auto& s : h->sigs) s.count = 0;
  for (int e = 0; e < n_entries; ++e) {
    const int s = slots_host[e], n = counts_host[e], base = h->len[s];
    for (auto& sg : h->sigs) {
      const int rows = n * sg.H;
      for (int r0 = 0; r0 < rows; r0 += sg.rpt) {
        m[sg.off_row0 + sg.count] = t * sg.H + r0;
        m[sg.off_rows + sg.count] = std::min(sg.rpt, rows - r0);
        m[sg.off_slot + sg.count] = s;
        ++sg.count;
      }
    }
    for (int i = 0; i < n; ++i, ++t) {
      m[h->off_tok + t] = tokens_host[t];
      m[h->off_slot + t] = s;
      m[h->off_pos + t] = base + i;
    }
    max_ctx = std::max(max_ctx, base + n);
  }
  for (int i = 0; i < n_want; ++i) m[h->off_want + i] = want_host[i];
  B200_CUDA(cudaMemcpyAsync(h->meta_dev, m, (size_t)h->meta_ints * sizeof(int), cudaMemcpyHostToDevice, h->stream));
  B200_CUDA(cudaEventRecord(h->ev_meta, h->stream));
  const int rc = h->f32 ? step_body<float>(h, t, n_want, max_ctx, logits_dev) : step_body<bf16>(h, t, n_want, max_ctx, logits_dev);
  if (rc != B200_OK) return rc;
  if (h->time_kernels && h->ev_used) {      // diagnostics only: waits for the step and sums its intervals per class
    B200_CUDA(cudaStreamSynchronize(h->stream));
    for (size_t i = 0; i + 1 < h->ev_used; i += 2) {
      float ms = 0.f;
      B200_CUDA(cudaEventElapsedTime(&ms, h->ev_pool[i], h->ev_pool[i + 1]));
      h->class_ms[h->ev_class[i]] += ms;
    }
    h->ev_used = 0;
  }
  for (int e = 0; e < n_entries; ++e) h->len[slots_host[e]] += counts_host[e];
  h->last_tokens = t; h->last_want = n_want;
  return B200_OK;
}

int b200_dlm_sample(b200_dlm* h, const float* noise_dev, int use_sampling, float temp, int top_k, int64_t* out_dev) {
  using namespace b200::lm;
  if (!h || !h->slots || h->last_want < 1 || !out_dev) B200_FAIL(B200_ERR_STATE, "dlm_sample: the last step left no logits");
  const int V = h->cfg.vocab;
  DeviceGuard g(h->device);
  if (!use_sampling || temp <= 0.f) {        // greedy: on the fp32 logits, whatever the vocabulary's size
    B200_LAUNCH(argmax_rows_kernel, h->last_want, 256, 0, h->stream, h->logits, V, reinterpret_cast<long long*>(out_dev));
    return check_launch("dlm_sample (greedy)");
  }
  if (V + 1 > 65535) B200_FAIL(B200_ERR_SHAPE, "dlm_sample: the sampler takes vocabularies up to 65534");
  if (top_k < 1) top_k = 1;
  if (top_k > SAMPLE_MAX_K) B200_FAIL(B200_ERR_SHAPE, "dlm_sample: top_k above %d", SAMPLE_MAX_K);
  if (!noise_dev) B200_FAIL(B200_ERR_INVALID, "dlm_sample: sampling needs noise");
  const long long n = (long long)h->last_want * V;
  B200_LAUNCH(logits_to_bf16_kernel, (unsigned)ceil_div64(n, 256), 256, 0, h->stream, h->logits, h->logits_bf, n);
  const int k = top_k < V ? top_k : V;
  B200_LAUNCH(sample_kernel, h->last_want, SAMPLE_THREADS, 0, h->stream, h->logits_bf, (long long)V, noise_dev, (long long)k,
              reinterpret_cast<long long*>(out_dev), V, use_sampling, temp, top_k);
  return check_launch("dlm_sample");
}

int b200_dlm_read_buffer(b200_dlm* h, const char* name, void* dst_dev, int64_t capacity_bytes, int64_t* nbytes) {
  if (!h || !h->slots || !name) B200_FAIL(B200_ERR_STATE, "dlm_read_buffer: no cache");
  DeviceGuard g(h->device);
  const std::string n(name);
  const size_t W = h->cfg.width;
  if (n == "logits") {
    const int64_t bytes = (int64_t)h->last_want * h->cfg.vocab * 4;
    if (nbytes) *nbytes = bytes;
    if (!dst_dev) return B200_OK;
    if (capacity_bytes < bytes) B200_FAIL(B200_ERR_SHAPE, "dlm_read_buffer: '%s' needs %lld bytes", name, (long long)bytes);
    B200_CUDA(cudaMemcpyAsync(dst_dev, h->logits, (size_t)bytes, cudaMemcpyDeviceToDevice, h->stream));
    return B200_OK;
  }
  if (n == "layers") {
    if (!h->trace) B200_FAIL(B200_ERR_STATE, "dlm_read_buffer: 'layers' needs option trace_layers = 1 before cache_begin");
    const int64_t row = (int64_t)h->last_tokens * W * 4;
    const int64_t bytes = row * h->cfg.n_layers;
    if (nbytes) *nbytes = bytes;
    if (!dst_dev) return B200_OK;
    if (capacity_bytes < bytes) B200_FAIL(B200_ERR_SHAPE, "dlm_read_buffer: '%s' needs %lld bytes", name, (long long)bytes);
    B200_CUDA(cudaMemcpy2DAsync(dst_dev, (size_t)row, h->trace, (size_t)h->tmax * W * 4, (size_t)row, (size_t)h->cfg.n_layers,
                                cudaMemcpyDeviceToDevice, h->stream));
    return B200_OK;
  }
  if (n == "error_flags") {
    if (nbytes) *nbytes = 4;
    if (!dst_dev) return B200_OK;
    if (capacity_bytes < 4) B200_FAIL(B200_ERR_SHAPE, "dlm_read_buffer: 'error_flags' needs 4 bytes");
    B200_CUDA(cudaMemcpyAsync(dst_dev, h->err, 4, cudaMemcpyDeviceToDevice, h->stream));
    return B200_OK;
  }
  B200_FAIL(B200_ERR_INVALID, "dlm_read_buffer: unknown buffer '%s'", name);
}

int b200_dlm_read_timers(b200_dlm* h, double* ms4_host, int reset) {
  if (!h || !ms4_host) B200_FAIL(B200_ERR_INVALID, "dlm_read_timers: null argument");
  for (int i = 0; i < 4; ++i) { ms4_host[i] = h->class_ms[i]; if (reset) h->class_ms[i] = 0; }
  return B200_OK;
}

// weights once + the cached latents the new tokens read + the latents they write
int64_t b200_dlm_algorithmic_bytes(b200_dlm* h, int tokens, int context) {
  if (!h) return 0;
  int64_t b = h->weight_bytes - (int64_t)h->cfg.vocab * h->cfg.width * esize(h);     // the embedding is gathered, not streamed
  for (auto& L : h->layers) b += ((int64_t)context + tokens) * L.c.kv_rank * esize(h);
  return b + (int64_t)tokens * h->cfg.width * esize(h);
}

// multiply-adds x 2 of the linears and of attention in the form the kernels run it (scores and sums against the latent)
int64_t b200_dlm_algorithmic_flops(b200_dlm* h, int tokens, int context) {
  if (!h) return 0;
  const int64_t T = tokens, W = h->cfg.width;
  int64_t f = 0;
  for (auto& L : h->layers) {
    const int64_t H = L.c.heads, dk = L.c.dim, dv = L.c.vdim, r = L.c.kv_rank;
    f += 2 * T * W * L.ncat + 2 * T * H * dk * r + 2 * T * H * dv * r + 2 * T * W * H * dv;
    if (L.c.mlp != B200_MLP_NONE) f += 2 * T * W * L.c.ff;
    f += 4 * H * r * (T * context + T * (T + 1) / 2);
  }
  return f + 2 * T * W * h->cfg.vocab;
}

int b200_op_latent_attention(const float* qa_dev, const void* latents_dev, int dtype, const float* sink_dev, float* out_dev,
                             int T, int H, int r, int pos0, int nsplit, int tensor_cores, void* stream) {
  if (!qa_dev || !latents_dev || !sink_dev || !out_dev) B200_FAIL(B200_ERR_INVALID, "op_latent_attention: null pointer");
  if (T < 1 || H < 1 || r < 1 || r > 1024 || pos0 < 0) B200_FAIL(B200_ERR_SHAPE, "op_latent_attention: bad shape");
  if (dtype != B200_F32 && dtype != B200_BF16) B200_FAIL(B200_ERR_INVALID, "op_latent_attention: latents must be f32 or bf16");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rpt = rows_per_tile(r), rows = T * H, tiles = ceil_div(rows, rpt);
  std::vector<int> meta((size_t)3 * tiles + T);
  for (int i = 0; i < tiles; ++i) { meta[i] = i * rpt; meta[tiles + i] = std::min(rpt, rows - i * rpt); meta[2 * tiles + i] = 0; }
  for (int t = 0; t < T; ++t) meta[3 * tiles + t] = pos0 + t;
  int* meta_dev = nullptr; float* part = nullptr;
  B200_CUDA(cudaMalloc(&meta_dev, meta.size() * sizeof(int)));
  B200_CUDA(cudaMemcpyAsync(meta_dev, meta.data(), meta.size() * sizeof(int), cudaMemcpyHostToDevice, st));
  AttnParams p;
  p.qa = qa_dev; p.cache = latents_dev; p.sink = sink_dev; p.tile_row0 = meta_dev; p.tile_rows = meta_dev + tiles; p.tile_slot = meta_dev + 2 * tiles;
  p.tok_pos = meta_dev + 3 * tiles; p.out = out_dev; p.cap = pos0 + T; p.r = r; p.H = H;
  const size_t part_floats = (size_t)600 * 16 * (r + 2);
  p.nsplit = pick_split(nsplit, tiles, pos0 + T, rpt, r, nsplit > 0 ? (size_t)tiles * nsplit * rpt * (r + 2) : part_floats);
  const size_t need = (size_t)tiles * p.nsplit * rpt * (r + 2);
  B200_CUDA(cudaMalloc(&part, std::max(need, (size_t)1) * sizeof(float)));
  p.part = part;
  int rc = dtype == B200_F32 ? run_attention<float>(st, p, tiles, rpt) : run_attention<bf16>(st, p, tiles, rpt, tensor_cores != 0);
  cudaError_t e = cudaStreamSynchronize(st);
  cudaFree(meta_dev); cudaFree(part);
  if (rc == B200_OK && e != cudaSuccess) { set_error("op_latent_attention: %s", cudaGetErrorString(e)); rc = B200_ERR_CUDA; }
  return rc;
}

}  // extern "C"
