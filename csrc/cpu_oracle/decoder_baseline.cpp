// A whole training step of the small pre-LN decoder, composed from the oracle's scalar kernels.
//
// The reference runs this model on its CPU backend as a chain of single-threaded scalar loops: one
// kernel per op, no fusion, naive ikj matmul (rumus/src/backend/cpu.rs, rumus/src/nn/transformer.rs,
// rumus/src/nn/attention.rs).  This file states the same chain in C++ over the oracle kernels
// of cpu_oracle.cpp, so that it serves two purposes:
//   * an independent end-to-end oracle for the framework's decoder (loss and every gradient), and
//   * the timed CPU baseline of the functional configuration (2 layers, d 128, 4 heads, FFN 512).
//
// Layout conventions: activations are token-major [N = batch*seq, d]; Linear weights are [in, out];
// parameters are held in the order of the framework's state dict so the Python side can copy a
// state dict in tensor by tensor.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

extern "C" {
void orc_add(const float*, const float*, float*, long long);
void orc_scale(const float*, float, float*, long long);
void orc_relu(const float*, float*, long long);
void orc_relu_backward(const float*, const float*, float*, long long);
void orc_matmul(const float*, const float*, float*, int, int, int);
void orc_bmm(const float*, const float*, float*, int, int, int, int);
void orc_add_bias(const float*, const float*, float*, int, int);
void orc_sum_rows(const float*, float*, int, int);
void orc_softmax(const float*, float*, int, int);
void orc_softmax_backward(const float*, const float*, float*, int, int);
void orc_layer_norm(const float*, const float*, const float*, float*, float*, int, int, float);
void orc_layer_norm_backward(const float*, const float*, const float*, const float*, float*, float*, float*, int, int);
void orc_embedding(const long long*, const float*, float*, long long, int);
void orc_embedding_backward(const long long*, const float*, float*, long long, int, int);
float orc_cross_entropy(const float*, const long long*, float*, int, int);
void orc_adam_step(float*, float*, float*, const float*, long long, float, float, float, float, float, float, float, int);
}

namespace {

using Buf = std::vector<float>;

struct Tensor {
  Buf p, g, m, v;
  explicit Tensor(long long n = 0) : p((size_t)n, 0.f), g((size_t)n, 0.f), m((size_t)n, 0.f), v((size_t)n, 0.f) {}
};

// indices into Layer::t
enum { LN1_W, LN1_B, WQ, BQ, WK, BK, WV, BV, WO, BO, LN2_W, LN2_B, W1, B1, W2, B2, LAYER_TENSORS };

struct LayerAct {
  Buf x_in, h1, ln1_save, q, k, v, qh, kh_t, vh, probs, oh, o, x_mid, h2, ln2_save, u, a;
};

struct Decoder {
  int vocab, seq, d, heads, layers, ffn, batch, hd, N;
  std::vector<Tensor> t;      // tok, pos, layers * LAYER_TENSORS, lnf_w, lnf_b, head
  std::vector<LayerAct> act;
  Buf x_final, hf, lnf_save, logits, dlogits;
  std::vector<long long> pos_idx;
  long long steps = 0;
  Tensor& lt(int l, int i) { return t[(size_t)(2 + l * LAYER_TENSORS + i)]; }
  Tensor& lnf_w() { return t[(size_t)(2 + layers * LAYER_TENSORS)]; }
  Tensor& lnf_b() { return t[(size_t)(2 + layers * LAYER_TENSORS + 1)]; }
  Tensor& head() { return t[(size_t)(2 + layers * LAYER_TENSORS + 2)]; }
};

void transpose(const float* a, float* o, int rows, int cols) {
  for (int i = 0; i < rows; ++i) for (int j = 0; j < cols; ++j) o[(long long)j * rows + i] = a[(long long)i * cols + j];
}

// [N, d] token-major -> [B*H, S, hd]
void split_heads(const Decoder& D, const float* x, float* o) {
  for (int b = 0; b < D.batch; ++b) for (int h = 0; h < D.heads; ++h) for (int s = 0; s < D.seq; ++s)
    std::memcpy(o + (((long long)b * D.heads + h) * D.seq + s) * D.hd,
                x + ((long long)b * D.seq + s) * D.d + h * D.hd, sizeof(float) * D.hd);
}
void merge_heads(const Decoder& D, const float* x, float* o) {
  for (int b = 0; b < D.batch; ++b) for (int h = 0; h < D.heads; ++h) for (int s = 0; s < D.seq; ++s)
    std::memcpy(o + ((long long)b * D.seq + s) * D.d + h * D.hd,
                x + (((long long)b * D.heads + h) * D.seq + s) * D.hd, sizeof(float) * D.hd);
}

// y = x W + b
void linear(const float* x, const Tensor& w, const Tensor& b, float* y, int n, int in, int out) {
  orc_matmul(x, w.p.data(), y, n, in, out);
  orc_add_bias(y, b.p.data(), y, n, out);
}
// dW = x^T dy, db = column sums of dy, dx = dy W^T
void linear_backward(const float* x, Tensor& w, Tensor* b, const float* dy, float* dx, int n, int in, int out,
                     Buf& scratch) {
  scratch.resize((size_t)std::max((long long)n * in, (long long)in * out));
  transpose(x, scratch.data(), n, in);                       // [in, n]
  orc_matmul(scratch.data(), dy, w.g.data(), in, n, out);
  if (b) orc_sum_rows(dy, b->g.data(), n, out);
  if (dx) {
    transpose(w.p.data(), scratch.data(), in, out);          // [out, in]
    orc_matmul(dy, scratch.data(), dx, n, out, in);
  }
}

float forward(Decoder& D, const long long* x, const long long* y) {
  const int N = D.N, d = D.d, S = D.seq, BH = D.batch * D.heads, hd = D.hd;
  Buf cur((size_t)N * d), tmp((size_t)N * d);
  orc_embedding(x, D.t[0].p.data(), cur.data(), N, d);
  orc_embedding(D.pos_idx.data(), D.t[1].p.data(), tmp.data(), N, d);
  orc_add(cur.data(), tmp.data(), cur.data(), (long long)N * d);
  const float scale = 1.f / std::sqrt((float)hd);
  for (int l = 0; l < D.layers; ++l) {
    LayerAct& A = D.act[(size_t)l];
    A.x_in = cur;
    orc_layer_norm(cur.data(), D.lt(l, LN1_W).p.data(), D.lt(l, LN1_B).p.data(), A.h1.data(), A.ln1_save.data(), N, d, 1e-5f);
    linear(A.h1.data(), D.lt(l, WQ), D.lt(l, BQ), A.q.data(), N, d, d);
    linear(A.h1.data(), D.lt(l, WK), D.lt(l, BK), A.k.data(), N, d, d);
    linear(A.h1.data(), D.lt(l, WV), D.lt(l, BV), A.v.data(), N, d, d);
    split_heads(D, A.q.data(), A.qh.data());
    split_heads(D, A.v.data(), A.vh.data());
    split_heads(D, A.k.data(), tmp.data());
    for (int i = 0; i < BH; ++i) transpose(tmp.data() + (long long)i * S * hd, A.kh_t.data() + (long long)i * S * hd, S, hd);
    // scores -> scale -> causal mask -> softmax (in A.probs)
    orc_bmm(A.qh.data(), A.kh_t.data(), A.probs.data(), BH, S, hd, S);
    orc_scale(A.probs.data(), scale, A.probs.data(), (long long)BH * S * S);
    for (int i = 0; i < BH; ++i) for (int r = 0; r < S; ++r) for (int c = r + 1; c < S; ++c)
      A.probs[((size_t)i * S + r) * S + c] = -1e30f;
    orc_softmax(A.probs.data(), A.probs.data(), BH * S, S);
    orc_bmm(A.probs.data(), A.vh.data(), A.oh.data(), BH, S, S, hd);
    merge_heads(D, A.oh.data(), A.o.data());
    linear(A.o.data(), D.lt(l, WO), D.lt(l, BO), tmp.data(), N, d, d);
    orc_add(cur.data(), tmp.data(), cur.data(), (long long)N * d);
    A.x_mid = cur;
    orc_layer_norm(cur.data(), D.lt(l, LN2_W).p.data(), D.lt(l, LN2_B).p.data(), A.h2.data(), A.ln2_save.data(), N, d, 1e-5f);
    linear(A.h2.data(), D.lt(l, W1), D.lt(l, B1), A.u.data(), N, d, D.ffn);
    orc_relu(A.u.data(), A.a.data(), (long long)N * D.ffn);
    linear(A.a.data(), D.lt(l, W2), D.lt(l, B2), tmp.data(), N, D.ffn, d);
    orc_add(cur.data(), tmp.data(), cur.data(), (long long)N * d);
  }
  D.x_final = cur;
  orc_layer_norm(cur.data(), D.lnf_w().p.data(), D.lnf_b().p.data(), D.hf.data(), D.lnf_save.data(), N, d, 1e-5f);
  orc_matmul(D.hf.data(), D.head().p.data(), D.logits.data(), N, d, D.vocab);
  return orc_cross_entropy(D.logits.data(), y, D.dlogits.data(), N, D.vocab);
}

void backward(Decoder& D, const long long* x) {
  const int N = D.N, d = D.d, S = D.seq, BH = D.batch * D.heads, hd = D.hd, f = D.ffn;
  const long long nd = (long long)N * d;
  const float scale = 1.f / std::sqrt((float)hd);
  Buf scratch, dcur((size_t)nd), dh((size_t)nd), t1((size_t)nd), t2((size_t)nd), t3((size_t)nd);
  Buf du((size_t)N * f), da((size_t)N * f);
  Buf dprobs((size_t)BH * S * S), dqh((size_t)nd), dkh((size_t)nd), dvh((size_t)nd), tr((size_t)BH * S * S);
  // head and final norm
  linear_backward(D.hf.data(), D.head(), nullptr, D.dlogits.data(), dh.data(), N, d, D.vocab, scratch);
  orc_layer_norm_backward(D.x_final.data(), D.lnf_w().p.data(), dh.data(), D.lnf_save.data(), dcur.data(),
                          D.lnf_w().g.data(), D.lnf_b().g.data(), N, d);
  for (int l = D.layers - 1; l >= 0; --l) {
    LayerAct& A = D.act[(size_t)l];
    // MLP branch: x_out = x_mid + W2 relu(W1 LN2(x_mid))
    linear_backward(A.a.data(), D.lt(l, W2), &D.lt(l, B2), dcur.data(), da.data(), N, f, d, scratch);
    orc_relu_backward(A.u.data(), da.data(), du.data(), (long long)N * f);
    linear_backward(A.h2.data(), D.lt(l, W1), &D.lt(l, B1), du.data(), dh.data(), N, d, f, scratch);
    orc_layer_norm_backward(A.x_mid.data(), D.lt(l, LN2_W).p.data(), dh.data(), A.ln2_save.data(), t1.data(),
                            D.lt(l, LN2_W).g.data(), D.lt(l, LN2_B).g.data(), N, d);
    orc_add(dcur.data(), t1.data(), dcur.data(), nd);
    // attention branch: x_mid = x_in + Wo attn(LN1(x_in))
    linear_backward(A.o.data(), D.lt(l, WO), &D.lt(l, BO), dcur.data(), t1.data(), N, d, d, scratch);
    split_heads(D, t1.data(), t2.data());                                   // d(oh) [BH, S, hd]
    // dV = P^T dO ; dP = dO V^T
    for (int i = 0; i < BH; ++i) transpose(A.probs.data() + (long long)i * S * S, tr.data() + (long long)i * S * S, S, S);
    orc_bmm(tr.data(), t2.data(), dvh.data(), BH, S, S, hd);
    for (int i = 0; i < BH; ++i) transpose(A.vh.data() + (long long)i * S * hd, t3.data() + (long long)i * S * hd, S, hd);
    orc_bmm(t2.data(), t3.data(), dprobs.data(), BH, S, hd, S);
    orc_softmax_backward(A.probs.data(), dprobs.data(), dprobs.data(), BH * S, S);
    orc_scale(dprobs.data(), scale, dprobs.data(), (long long)BH * S * S);
    // dQ = dS K ; dK = dS^T Q   (K row-major is the transpose of kh_t)
    for (int i = 0; i < BH; ++i) transpose(A.kh_t.data() + (long long)i * S * hd, t3.data() + (long long)i * S * hd, hd, S);
    orc_bmm(dprobs.data(), t3.data(), dqh.data(), BH, S, S, hd);
    for (int i = 0; i < BH; ++i) transpose(dprobs.data() + (long long)i * S * S, tr.data() + (long long)i * S * S, S, S);
    orc_bmm(tr.data(), A.qh.data(), dkh.data(), BH, S, S, hd);
    // back through the three projections; their input gradients add up
    merge_heads(D, dqh.data(), t1.data());
    linear_backward(A.h1.data(), D.lt(l, WQ), &D.lt(l, BQ), t1.data(), dh.data(), N, d, d, scratch);
    merge_heads(D, dkh.data(), t1.data());
    linear_backward(A.h1.data(), D.lt(l, WK), &D.lt(l, BK), t1.data(), t2.data(), N, d, d, scratch);
    orc_add(dh.data(), t2.data(), dh.data(), nd);
    merge_heads(D, dvh.data(), t1.data());
    linear_backward(A.h1.data(), D.lt(l, WV), &D.lt(l, BV), t1.data(), t2.data(), N, d, d, scratch);
    orc_add(dh.data(), t2.data(), dh.data(), nd);
    orc_layer_norm_backward(A.x_in.data(), D.lt(l, LN1_W).p.data(), dh.data(), A.ln1_save.data(), t1.data(),
                            D.lt(l, LN1_W).g.data(), D.lt(l, LN1_B).g.data(), N, d);
    orc_add(dcur.data(), t1.data(), dcur.data(), nd);
  }
  orc_embedding_backward(x, dcur.data(), D.t[0].g.data(), N, d, D.vocab);
  orc_embedding_backward(D.pos_idx.data(), dcur.data(), D.t[1].g.data(), N, d, D.seq);
}

}  // namespace

extern "C" {

void* orc_decoder_create(int vocab, int seq, int d, int heads, int layers, int ffn, int batch) {
  if (vocab <= 0 || seq <= 0 || d <= 0 || heads <= 0 || d % heads || layers < 0 || ffn <= 0 || batch <= 0) return nullptr;
  Decoder* D = new Decoder;
  D->vocab = vocab; D->seq = seq; D->d = d; D->heads = heads; D->layers = layers; D->ffn = ffn; D->batch = batch;
  D->hd = d / heads; D->N = batch * seq;
  D->t.emplace_back((long long)vocab * d);
  D->t.emplace_back((long long)seq * d);
  for (int l = 0; l < layers; ++l) {
    const long long sizes[LAYER_TENSORS] = {d, d, (long long)d * d, d, (long long)d * d, d, (long long)d * d, d,
                                            (long long)d * d, d, d, d, (long long)d * ffn, ffn, (long long)ffn * d, d};
    for (long long s : sizes) D->t.emplace_back(s);
  }
  D->t.emplace_back(d); D->t.emplace_back(d); D->t.emplace_back((long long)d * vocab);
  const size_t nd = (size_t)D->N * d, nf = (size_t)D->N * ffn, bss = (size_t)batch * heads * seq * seq;
  D->act.resize((size_t)layers);
  for (auto& A : D->act) {
    for (Buf* b : {&A.h1, &A.q, &A.k, &A.v, &A.qh, &A.kh_t, &A.vh, &A.oh, &A.o, &A.h2}) b->assign(nd, 0.f);
    A.ln1_save.assign((size_t)D->N * 2, 0.f); A.ln2_save.assign((size_t)D->N * 2, 0.f);
    A.probs.assign(bss, 0.f); A.u.assign(nf, 0.f); A.a.assign(nf, 0.f);
  }
  D->hf.assign(nd, 0.f); D->lnf_save.assign((size_t)D->N * 2, 0.f);
  D->logits.assign((size_t)D->N * vocab, 0.f); D->dlogits.assign((size_t)D->N * vocab, 0.f);
  D->pos_idx.resize((size_t)D->N);
  for (int i = 0; i < D->N; ++i) D->pos_idx[(size_t)i] = i % seq;
  return D;
}

int orc_decoder_num_tensors(void* h) { return (int)static_cast<Decoder*>(h)->t.size(); }

// which: 0 parameter, 1 gradient, 2 Adam first moment, 3 Adam second moment
float* orc_decoder_tensor(void* h, int i, int which, long long* numel) {
  Decoder* D = static_cast<Decoder*>(h);
  if (i < 0 || i >= (int)D->t.size()) return nullptr;
  Tensor& t = D->t[(size_t)i];
  if (numel) *numel = (long long)t.p.size();
  return which == 0 ? t.p.data() : which == 1 ? t.g.data() : which == 2 ? t.m.data() : t.v.data();
}

// x, y: [batch*seq] token ids.  Returns the mean cross entropy; with `with_backward` every gradient
// is (re)written.
float orc_decoder_forward_backward(void* h, const long long* x, const long long* y, int with_backward) {
  Decoder* D = static_cast<Decoder*>(h);
  for (int i = 0; i < D->N; ++i)
    if (x[i] < 0 || x[i] >= D->vocab || y[i] < 0 || y[i] >= D->vocab) return NAN;
  const float loss = forward(*D, x, y);
  if (with_backward) backward(*D, x);
  return loss;
}

void orc_decoder_adam(void* h, float lr, float b1, float b2, float eps) {
  Decoder* D = static_cast<Decoder*>(h);
  D->steps++;
  const float bc1 = 1.f - std::pow(b1, (float)D->steps), bc2 = 1.f - std::pow(b2, (float)D->steps);
  for (auto& t : D->t)
    orc_adam_step(t.p.data(), t.m.data(), t.v.data(), t.g.data(), (long long)t.p.size(), lr, b1, b2, eps, bc1, bc2, 0.f, 0);
}

void orc_decoder_destroy(void* h) { delete static_cast<Decoder*>(h); }
}
