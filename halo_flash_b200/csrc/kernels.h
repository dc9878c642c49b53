// Internal launch interface between the C ABI (api.cu) and the kernel files.
// Launchers validate nothing: api.cu has already checked pointers, sizes and
// alignment and set `vec` (16-byte vector path) or cleared it (scalar path).
// Each returns the cudaError_t of its launch.
#ifndef HALO_B200_KERNELS_H_
#define HALO_B200_KERNELS_H_

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <utility>

namespace halo_b200 {

// True unless halo_b200_tune("pdl", 0) switched programmatic dependent launch off.
bool PdlEnabled();

// Every kernel launch of the library: a plain stream-ordered launch that additionally allows the
// kernel to be scheduled while its predecessor in the stream drains (the kernels order
// themselves with pdl_begin()). Safe next to foreign kernels: one that never signals lets its
// successor start only at its completion, and a successor launched without the attribute waits
// for full completion as usual. Capturable into CUDA graphs (a programmatic edge).
template <typename... KArgs, typename... Args>
inline cudaError_t LaunchKernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = PdlEnabled() ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2 };
inline std::size_t DTypeSize(int t) { return t == kF32 ? 4 : 2; }

// Where a token's position comes from (group 3). pos = base * scale, base =
// params[t * pstride + slot] when params is set, else pos0 + t (uint32 wrap-around
// arithmetic, as src/kernels/core.hip:289-311 computes it).
struct PosSpec {
  const uint32_t* params = nullptr;
  uint32_t pstride = 0, slot = 0;
  uint32_t pos0 = 0, scale = 1;
};

constexpr int kMaxRotHalf = 128;  // inverse-frequency table travels as a kernel argument
struct InvFreq {
  float f[kMaxRotHalf];
};

// ---- groups 1 and 2 (L2): row norms ------------------------------------------------
// One kernel family covers RMSNorm, residual-add + RMSNorm, L2 norm and the Q8
// epilogues. Row r lives at base + (r / rows_per_entry) * entry_stride +
// (r % rows_per_entry) * d elements; dense tensors use rows_per_entry = rows.
struct NormArgs {
  const void* x = nullptr;      // [rows][d] x_dtype
  int x_dtype = kF32;
  const void* delta = nullptr;  // optional, x_dtype, dense [rows][d]: x + delta is normalized
  void* res = nullptr;          // with delta: the sum is stored here in x_dtype (may alias x)
  const float* w = nullptr;     // gamma rows (fp32) or null
  uint32_t w_stride = 0, w_period = 1;
  int one_plus = 0;             // multiply by (1 + w) instead of w
  void* y = nullptr;            // normalized rows in y_dtype, or null (may alias x)
  int y_dtype = kF32;
  void* y16 = nullptr;          // optional extra fp16 copy (the reference's *_h kernels)
  uint32_t y16_tokens = 0;      // > 0: y16 is K-blocked [cols / 64][tokens][64]
  uint8_t* q8_0 = nullptr;      // optional Q8_0 rows, d / 32 blocks of 34 bytes
  int8_t* xq = nullptr;         // optional int8 activation codes
  float* xd = nullptr;          //   and their fp32 scales
  uint32_t kb_tokens = 0;       // > 0: xq / xd K-blocked [cols / 64][tokens][64], [cols / 32][tokens]
  uint32_t kb_period = 1;       // rows per token in the K-blocked layouts (column = (r % period) * d + i)
  float* rscale = nullptr;      // optional per-row scale
  uint32_t d = 0, rows = 0;
  float eps = 0.0f;
  int l2 = 0;                   // 1: scale = 1 / sqrt(ss + eps) (no mean, no gamma)
  uint32_t rows_per_entry = 0;  // 0 = dense
  uint64_t entry_stride = 0;
  int threads_per_row = 0;      // 0 = pick automatically
  int short_rows_k1 = 0;        // 1: rows of <= 32 octets keep one octet per thread (default two)
  int force_general = 0;        // 1: never take the lean kernel (tests compare the two)
  int keep_hint = 1;            // 0: the add + norm stores its residual without the L2 keep policy
  bool vec = true;
};
cudaError_t LaunchNorm(const NormArgs& a, cudaStream_t s);
// The lean kernel with three or five octets per thread (rows of 3 g / 5 g octets, g = 1 << lg threads per row; five
// only for 16-bit rows), for the (x, y) type pairs the lean kernels exist for; called by LaunchNorm.
cudaError_t LaunchNormLeanOdd(const NormArgs& a, unsigned lg, int k, unsigned rows_per_cta, unsigned grid, cudaStream_t s);

// ---- group 2: gated RMSNorm --------------------------------------------------------
struct GatedArgs {
  const void* o = nullptr;
  int o_dtype = kF32;
  const void* z = nullptr;
  int z_dtype = kF32;
  const float* w = nullptr;  // [d], shared by every row
  void* y = nullptr;         // may alias o
  int y_dtype = kF32;
  uint32_t d = 0, rows = 0;
  float eps = 0.0f;
  uint32_t mode = 0;  // 0 SiLU(z), 1 sigmoid(z)
  int threads_per_row = 0;
  int short_rows_k1 = 0;
  int rows_per_group = 0;  // 2: short rows keep two rows per thread group in flight
  int force_general = 0;   // 1: never take the lean kernel (tests compare the two)
  bool vec = true;
};
cudaError_t LaunchGatedNorm(const GatedArgs& a, cudaStream_t s);

// ---- group 3: rotary embedding --------------------------------------------------------
struct RopeArgs {
  void* x = nullptr;  // [tokens][heads][hd], in place
  int dtype = kF32;
  uint32_t tokens = 0, heads = 0, hd = 0, rot = 0;
  uint64_t token_stride = 0;  // elements between tokens
  void* x2 = nullptr;         // optional second tensor rotated with the same positions (K beside Q)
  uint32_t heads2 = 0;
  uint64_t token_stride2 = 0;
  PosSpec pos;
  uint32_t* pos_out = nullptr;  // optional [tokens]: the position each token used
  bool vec = true;
};
cudaError_t LaunchRope(const RopeArgs& a, const InvFreq& f, cudaStream_t s);

// RMSNorm (shared gamma) + RoPE on rows of d <= 2048 (one row = one head of one
// token), optionally de-interleaving a [rows][2 * d] q|gate input and appending
// the rotated row to a cache.
struct NormRopeArgs {
  const void* in = nullptr;
  int in_dtype = kF32;
  uint64_t in_row_stride = 0;  // elements between input rows (d, or 2 * d for q|gate)
  void* out = nullptr;         // [rows][d] out_dtype, may alias in when in_row_stride == d
  int out_dtype = kF32;
  void* gate = nullptr;        // optional [rows][d] in_dtype copy of in[row][d .. 2d)
  void* cache = nullptr;       // optional [rows][d] out_dtype second copy of the result
  const float* w = nullptr;    // [d] or null (no norm: split + rope only)
  int one_plus = 0;
  float eps = 0.0f;
  uint32_t d = 0, rot = 0, heads = 0, rows = 0;
  // Optional second tensor with its own gamma, normalized and rotated in the same launch with
  // the same positions (K beside Q): token t owns rows [t * heads2, (t + 1) * heads2) of it.
  const void* in2 = nullptr;
  uint64_t in_row_stride2 = 0;
  void* out2 = nullptr;
  void* cache2 = nullptr;
  const float* w2 = nullptr;
  uint32_t heads2 = 0;
  PosSpec pos;
  uint32_t* pos_out = nullptr;  // optional [rows / heads]
  // Optional precomputed rotation table [tokens][2][rot / 2] fp32 (cos row, then sin row, per token;
  // LaunchRopeTable fills it). With it the kernel computes no sincosf, uses no shared memory and
  // has no barrier; pos / pos_out / the inverse frequencies are then unused.
  const float* table = nullptr;
  int rows_per_group = 0;       // rows a thread group keeps in flight: 2 (default) or 4
  int lean_k = 0;               // tuning: octets per lane of the lean kernel, 1 or 2 (0 = built-in choice)
  int staged = 1;               // 0: the lean kernel never stages rows in shared memory (tuning)
  int force_general = 0;        // 1: never take the lean kernel (tests compare the two)
};
cudaError_t LaunchNormRope(const NormRopeArgs& a, const InvFreq& f, cudaStream_t s);
// Validates the arguments of the Q + K fused norm + RoPE without launching anything: 0 = the vector kernels (and so
// the rotation-table form) can run them, 1 = valid but only the unfused fallback can (unaligned rows), -1 = invalid
// (message in err).
int CheckNormRopeQk(const void* q_in, uint64_t q_row_stride, void* q_out, void* q_gate, const float* w_q, uint32_t q_heads,
                    const void* k_in, void* k_out, void* k_cache, const float* w_k, uint32_t k_heads, int in_dtype,
                    int out_dtype, uint32_t d, uint32_t rotary_dim, uint32_t tokens, float theta, char* err,
                    size_t errlen);

// cos / sin of float(pos) * inv_freq[i] for every token: table[t][0][i] = cos, table[t][1][i] = sin.
struct RopeTableArgs {
  float* table = nullptr;
  uint32_t tokens = 0, rot = 0;
  PosSpec pos;
  uint32_t* pos_out = nullptr;
};
cudaError_t LaunchRopeTable(const RopeTableArgs& a, const InvFreq& f, cudaStream_t s);

struct SplitArgs {  // halo_split_qgate: [rows][2 * hd] -> q, gate
  const void* qg = nullptr;
  void* q = nullptr;
  void* gate = nullptr;
  int dtype = kF32;
  uint32_t hd = 0, rows = 0;
  uint32_t rows_per_entry = 0;  // 0 = dense
  uint64_t qg_entry_stride = 0, q_entry_stride = 0;
};
cudaError_t LaunchSplitQgate(const SplitArgs& a, cudaStream_t s);

// ---- group 4: elementwise ------------------------------------------------------------
enum EltOp : int { kOpSiluMul = 0, kOpAdd = 1, kOpAxpy = 2, kOpSigmoidGate = 3 };
constexpr int kMaxSegments = 4;
// One launch covers up to kMaxSegments independent tensors (e.g. the shared-expert and the
// routed-expert gate/up rows of a MoE layer): small tensors stop paying a launch of their own.
struct EltSegment {
  const void* a = nullptr;  // g (SiLU argument) / y (accumulator) / x
  const void* b = nullptr;  // up / x / gate
  void* y = nullptr;        // may alias a
  uint64_t n = 0;           // elements
};
struct EltArgs {
  int op = kOpSiluMul;
  int nseg = 1;
  EltSegment seg[kMaxSegments];
  int in_dtype = kF32;
  int y_dtype = kF32;
  float alpha = 1.0f;  // axpy
  bool vec = true;     // every segment 16-byte aligned
};
cudaError_t LaunchElementwise(const EltArgs& a, cudaStream_t s);

// ---- group 5: Q8_0 embedding gather ---------------------------------------------------
struct EmbedArgs {
  const uint8_t* table = nullptr;  // [vocab][row_bytes]
  uint64_t row_bytes = 0;
  uint32_t cols = 0;
  const uint32_t* ids = nullptr;  // token t at ids[t * id_stride + id_slot]; null: `token`
  uint32_t id_stride = 1, id_slot = 0;
  uint32_t token = 0;
  uint32_t tokens = 1;
  uint32_t vocab = 0;  // > 0: ids >= vocab produce a zero row instead of an out-of-range read
  void* out = nullptr;  // [tokens][cols]
  int out_dtype = kF32;
  bool vec = true;
  bool direct = true;  // tuning: rows read straight into registers where their shape allows (embed.cu)
};
cudaError_t LaunchEmbedQ8_0(const EmbedArgs& a, cudaStream_t s);

// ---- Q8 quantizers -------------------------------------------------------------------------
struct QuantArgs {
  const void* x = nullptr;  // row r at x + r * x_stride
  int x_dtype = kF32;
  uint64_t x_stride = 0;
  uint32_t cols = 0, rows = 0;
  uint8_t* q8_0 = nullptr;  // true Q8_0 rows
  int8_t* xq = nullptr;     // int8 activation form
  float* xd = nullptr;
  uint32_t kb_tokens = 0;   // > 0: K-blocked
  int8_t* xq2 = nullptr;    // optional second (residual) level, row-major only
  float* xd2 = nullptr;
  // optional product in front of the quantizer: v = (x * pre_scale[row][c / pre_h]) * pre_w[c], also stored to xn
  const float* pre_scale = nullptr;
  const float* pre_w = nullptr;
  uint32_t pre_h = 0;
  float* xn = nullptr;
  bool vec = true;
};
cudaError_t LaunchQuantize(const QuantArgs& a, cudaStream_t s);


// Hyper-connection residual (hc streams of h per token): combine + grouped RMSNorm and the
// elementwise stream ops around it (src/kernels/core.hip:601-625, 4105-4496, 4634-4714).
struct HcArgs {
  void* res;            // [tokens][hc][h], res_dtype; updated in place
  const void* out;      // [tokens][h], out_dtype (null when the block output is built from the experts)
  const float* inject;  // [tokens][hc] scatter logits
  const float* w;       // [hc][h] gammas
  void* y;              // [tokens][hc][h], y_dtype; may be null
  void* y16;            // fp16 copy; row-major, or K-blocked [hc h / 64][y16_tokens][64]; may be null
  float* rscale;        // [tokens][hc] row scales; may be null
  const float* iw;      // [irows][hc h] fp32 rows whose partial products with y go to ipart; may be null
  float* ipart;         // [tokens][hc][irows]
  int8_t* yq;           // K-blocked int8 copy [hc h / 64][y16_tokens][64]; may be null
  float* yd;            // its scales [hc h / 32][y16_tokens]
  // block output built in the kernel: sum over k slots of mw * yp[pos] + sigmoid(sg) * sx
  const void* yp;       // expert output rows [pairs][h], out_dtype (fp16 in the reference)
  const uint32_t* pos;  // [tokens][k] row of yp holding (token, slot)
  const float* mw;      // [tokens][k] routing weights
  const void* sx;       // [tokens][h] shared-expert output, fp32 or out_dtype
  const float* sg;      // [tokens] shared-expert gate logit
  uint32_t k;
  int sx_is_f32;
  uint32_t hc, h, tokens, irows, y16_tokens;
  float eps;
  int one_plus;
  int res_dtype, out_dtype, y_dtype;
  int vec;
  int fused_inject;  // tuning: 1 = the partial products are always computed inside the combine kernel
  int token_k;    // tuning: 2 = token-level shapes take two octets per stream per thread where they fit
  int row_level;  // tuning: 1 = one thread group per (token, stream) row even where a token-level shape exists
};
cudaError_t LaunchHcCombineNorm(const HcArgs& a, cudaStream_t s);

enum HcEltOp : int {
  kHcCombine = 0,     // res[t][s][i] += out[t][i] * 2 sigmoid(inject[t][s] / hc)
  kHcBroadcast = 1,   // res[t][s][i] = x[t][i]
  kHcMix = 2,         // mixed[t][i] = (sum_s xn[t][s][i] * sigmoid(gate[t][s][i])) / hc
  kAxpySigmoidRows = 3,  // y[t][i] += sigmoid(g[t]) * x[t][i]
  kInjectReduce = 4,  // inject[t][r] = sum_s ipart[(t hc + s) irows + r]
  kHcNormScales = 5,  // scale[row] = 1 / sqrt(mean(res_row^2) + eps)
  kScaleSilu = 6,     // a[i] = SiLU(b[i] * alpha)
};
struct HcEltArgs {
  int op;
  void* a;        // res / mixed / y / inject / scale (written)
  const void* b;  // out / x / xn / ipart / res
  const void* c;  // inject / gate / g
  int a_dtype, b_dtype;
  uint32_t hc, h, tokens, irows;
  float eps;
  int vec;
  const uint32_t* at_params;  // kHcBroadcast: the destination starts at a + at_params[at_slot] * at_stride elements
  uint32_t at_slot, at_stride;
  float alpha;
};
cudaError_t LaunchHcElt(const HcEltArgs& a, cudaStream_t s);

// Row append for `entries` sessions in one launch (src/kernels/batch_decode.hip:1700-1707): entry e copies
// src[e * src_stride ..+ n] to row params[e * pstride + slot] (rows `stride` elements apart) of the buffer whose
// device address is tab[e * tstride + tslot].
struct CopyAtArgs {
  const uint64_t* tab;
  uint32_t tstride, tslot;
  const float* src;
  const uint32_t* params;
  uint32_t slot, stride, n, src_stride, pstride, entries;
  int dst_dtype;
};
cudaError_t LaunchCopyAtEntries(const CopyAtArgs& a, cudaStream_t s);

// Causal depthwise conv + SiLU + per-head L2 norm of a Gated DeltaNet layer (src/kernels/core.hip:
// 445-456, 3002-3028, 3486-3611).
struct ConvArgs {
  const void* in;   // [tokens][channels], in_dtype
  float* state;     // [kern - 1][channels] fp32, oldest first; read by the conv, written by the advance
  const float* w;   // [channels][kern]
  void* out;        // [tokens][channels], out_dtype
  uint32_t channels, kern, l2_channels, d, tokens;
  float eps;
  int in_dtype, out_dtype;
  int vec;
  int tile;    // tuning: tokens per thread of the register form, 4 or 8 (0 = built-in choice)
  int staged;  // 1 = rows staged in shared memory by bulk asynchronous copies; 0 = rows held in registers
  // decode step over `entries` sessions in one launch (LaunchConvStep): entry e reads in + e * entry_stride, writes
  // out + e * entry_stride, and owns the state whose device address is state_tab[e * tstride + tslot]
  // (state_tab == NULL: one entry, `state`)
  const uint64_t* state_tab;
  uint32_t tstride, tslot, entries;
  uint64_t entry_stride;
};
cudaError_t ReadConvStageTimeouts(unsigned int* out);
cudaError_t ReadRopeStageTimeouts(unsigned int* out);
cudaError_t LaunchConvStep(const ConvArgs& a, cudaStream_t s);
cudaError_t LaunchConvL2norm(const ConvArgs& a, cudaStream_t s);
cudaError_t LaunchConvStateAdvance(const ConvArgs& a, cudaStream_t s);


// out[t] = sum over k slots, in order, of mw[t k + s] * yp[pos[t k + s]] (+ sigmoid(sg[t]) * sx[t]): the routed
// experts' outputs combined per token, optionally with the gated shared expert (src/kernels/core.hip:2372-2380,
// 5456-5480). pos == NULL: slot s of token t is row t k + s of yp.
struct MoeCombineArgs {
  const void* yp;       // [rows][n], yp_dtype
  const uint32_t* pos;  // [tokens][k] or NULL
  const float* mw;      // [tokens][k]
  const void* sx;       // [tokens][n] shared-expert output (fp32, or yp_dtype when sx_is_f32 == 0); NULL: none
  const float* sg;      // [tokens] gate logits
  void* out;            // [tokens][n], out_dtype
  uint32_t k, n, tokens;
  int yp_dtype, out_dtype, sx_is_f32;
  int accumulate;       // 1: out += (halo_axpy_slot), 0: out =
  int vec;
};
cudaError_t LaunchMoeCombine(const MoeCombineArgs& a, cudaStream_t s);


}  // namespace halo_b200

#endif  // HALO_B200_KERNELS_H_
