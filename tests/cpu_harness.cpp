// CPU build of the per-edge / per-atom arithmetic headers used by the CUDA
// kernels, exposed with a C ABI so pytest can check them against the oracle
// with ctypes.  Test infrastructure only: nothing in the product links this.
#include <cstring>
#include "../tace_b200/csrc/tace_math.cuh"
#include "../tace_b200/csrc/tp_gen.cuh"

using namespace tace;

#define TP_CASE(TAG)                                                                              \
  {                                                                                               \
    using TP = TPX_##TAG;                                                                         \
    double YY[TP::D], xx[TP::NX], ww[TP::NP];                                                     \
    alignas(16) double G[TP::NG];                                                                 \
    memcpy(YY, Y, sizeof YY); memcpy(xx, x, sizeof xx); memcpy(ww, w, sizeof ww);                 \
    TP::build_G<double>(YY, G);                                                                   \
    if (mode == 0) {                                                                              \
      double a0[TP::NMG0], w0[TP::NPG0];                                                          \
      memset(a0, 0, sizeof a0); memcpy(w0, ww + TP::P00, sizeof w0);                              \
      TP::fwd0<double>(xx, G, w0, a0); memcpy(out0 + TP::M00, a0, sizeof a0);                     \
      if (TP::NGRP > 1) {                                                                         \
        double a1[TP::NMG1], w1[TP::NPG1];                                                        \
        memset(a1, 0, sizeof a1); memcpy(w1, ww + TP::P01, sizeof w1);                            \
        TP::fwd1<double>(xx, G, w1, a1); memcpy(out0 + TP::M01, a1, sizeof a1);                   \
      }                                                                                           \
    } else {                                                                                      \
      double dw[TP::NP], dY[TP::D], dx[TP::NX];                                                   \
      memset(dY, 0, sizeof dY); memset(dx, 0, sizeof dx);                                         \
      TP::bwd<double>(xx, g, 1, G, ww, dw, dY, dx);                                               \
      memcpy(out0, dw, sizeof dw); memcpy(out1, dY, sizeof dY); memcpy(out2, dx, sizeof dx);      \
    }                                                                                             \
    return 0;                                                                                     \
  }

// What the kernels' weight accessors rely on: the generated backward code asks for the weight of path p exactly once,
// hands back its gradient before it asks for the next one, and walks the paths in ascending order.
struct OrderedWeights {
  const double* w;
  double* dw;
  int next_get = 0, next_put = 0, bad = 0;
  template <int P> double get() { if (P != next_get || next_put != P) ++bad; ++next_get; return w[P]; }
  template <int P> void put(double v) { if (P != next_put || next_get != P + 1) ++bad; ++next_put; dw[P] = v; }
};
#define TP_ORDER_CASE(TAG)                                                                        \
  {                                                                                               \
    using TP = TPX_##TAG;                                                                         \
    double YY[TP::D], xx[TP::NX], dY[TP::D], dx[TP::NX];                                          \
    alignas(16) double G[TP::NG];                                                                 \
    memcpy(YY, Y, sizeof YY); memcpy(xx, x, sizeof xx);                                           \
    memset(dY, 0, sizeof dY); memset(dx, 0, sizeof dx);                                           \
    TP::build_G<double>(YY, G);                                                                   \
    OrderedWeights wf{w, out0};                                                                   \
    TP::bwd_w<double>(xx, g, 1, G, wf, dY, dx);                                                   \
    memcpy(out1, dY, sizeof dY); memcpy(out2, dx, sizeof dx);                                     \
    return wf.bad + (wf.next_get != TP::NP) + (wf.next_put != TP::NP);                            \
  }

extern "C" {

// The backward pass through an accessor that counts every call out of order (return value; 0 = contract kept):
// out0 = d/dw, out1 = d/dY, out2 = d/dx as in h_tp mode 1.
int h_tp_bwd_ordered(int L, int Lin, const double* x, const double* Y, const double* w, const double* g,
                     double* out0, double* out1, double* out2) {
  if (L == 1 && Lin < 0) TP_ORDER_CASE(L1_S)
  if (L == 1 && Lin == 1) TP_ORDER_CASE(L1_F)
  if (L == 2 && Lin < 0) TP_ORDER_CASE(L2_S)
  if (L == 2 && Lin == 1) TP_ORDER_CASE(L2_N1)
  if (L == 2 && Lin == 2) TP_ORDER_CASE(L2_F)
  if (L == 3 && Lin < 0) TP_ORDER_CASE(L3_S)
  if (L == 3 && Lin == 1) TP_ORDER_CASE(L3_N1)
  if (L == 3 && Lin == 2) TP_ORDER_CASE(L3_N2)
  if (L == 3 && Lin == 3) TP_ORDER_CASE(L3_F)
  return -1;
}

// mode 0: forward (out0 = message components); mode 1: out0 = d/dw, out1 = d/dY, out2 = d/dx
// Lin: rank of the source features, or < 0 for the scalar source of the first layer
int h_tp(int L, int Lin, int mode, const double* x, const double* Y, const double* w, const double* g,
         double* out0, double* out1, double* out2) {
  if (L == 1 && Lin < 0) TP_CASE(L1_S)
  if (L == 1 && Lin == 1) TP_CASE(L1_F)
  if (L == 2 && Lin < 0) TP_CASE(L2_S)
  if (L == 2 && Lin == 1) TP_CASE(L2_N1)
  if (L == 2 && Lin == 2) TP_CASE(L2_F)
  if (L == 3 && Lin < 0) TP_CASE(L3_S)
  if (L == 3 && Lin == 1) TP_CASE(L3_N1)
  if (L == 3 && Lin == 2) TP_CASE(L3_N2)
  if (L == 3 && Lin == 3) TP_CASE(L3_F)
  return -1;
}

int h_tp_dims(int L, int Lin, int* dims) {
#define DIMS(TAG) { dims[0] = TPX_##TAG::NP; dims[1] = TPX_##TAG::NX; dims[2] = TPX_##TAG::NM; dims[3] = TPX_##TAG::D; return 0; }
  if (L == 1 && Lin < 0) DIMS(L1_S)
  if (L == 1 && Lin == 1) DIMS(L1_F)
  if (L == 2 && Lin < 0) DIMS(L2_S)
  if (L == 2 && Lin == 1) DIMS(L2_N1)
  if (L == 2 && Lin == 2) DIMS(L2_F)
  if (L == 3 && Lin < 0) DIMS(L3_S)
  if (L == 3 && Lin == 1) DIMS(L3_N1)
  if (L == 3 && Lin == 2) DIMS(L3_N2)
  if (L == 3 && Lin == 3) DIMS(L3_F)
  return -1;
}

#define PB_CASE(TAG)                                                                 \
  {                                                                                  \
    double aa[PB_##TAG::D], bb[PB_##TAG::NB], da[PB_##TAG::D];                       \
    memcpy(aa, a, sizeof aa);                                                        \
    if (mode == 0) { pb_fwd_##TAG<double>(aa, bb); memcpy(out, bb, sizeof bb); }     \
    else { memcpy(bb, db, sizeof bb); memset(da, 0, sizeof da);                      \
           pb_bwd_##TAG<double>(aa, bb, da); memcpy(out, da, sizeof da); }           \
    return PB_##TAG::NB;                                                             \
  }

// mode 0: b = A x A (out = b); mode 1: da from db.  Returns the number of b components.
// Lout: highest output rank, or < 0 for scalar outputs only.
int h_pb(int L, int Lout, int mode, const double* a, const double* db, double* out) {
  if (L == 1 && Lout < 0) PB_CASE(L1_T)
  if (L == 1 && Lout == 1) PB_CASE(L1_A)
  if (L == 2 && Lout < 0) PB_CASE(L2_T)
  if (L == 2 && Lout == 1) PB_CASE(L2_N1)
  if (L == 2 && Lout == 2) PB_CASE(L2_A)
  if (L == 3 && Lout < 0) PB_CASE(L3_T)
  if (L == 3 && Lout == 1) PB_CASE(L3_N1)
  if (L == 3 && Lout == 2) PB_CASE(L3_N2)
  if (L == 3 && Lout == 3) PB_CASE(L3_A)
  return -1;
}

#define PB3_CASE(TAG)                                                                          \
  {                                                                                            \
    using P = PB3X_##TAG;                                                                      \
    double aa[P::D], b2[P::NB2];                                                               \
    memcpy(aa, a, sizeof aa); memcpy(b2, b2in, sizeof b2);                                     \
    if (mode == 0) P::fwd<double>(aa, b2, out0, 1);                                            \
    else {                                                                                     \
      double db2[P::NB2], da[P::D];                                                            \
      memset(db2, 0, sizeof db2); memset(da, 0, sizeof da);                                    \
      P::bwd_b2<double>(aa, db3, 1, db2); P::bwd_a<double>(b2, db3, 1, da);                    \
      memcpy(out0, db2, sizeof db2); memcpy(out1, da, sizeof da);                              \
    }                                                                                          \
    return P::NB;                                                                              \
  }

// Third-order basis: mode 0: out0 = (b2 x a); mode 1: out0 = d/db2, out1 = d/da from db3.  Returns the number of
// third-order components.
int h_pb3(int L, int Lout, int mode, const double* a, const double* b2in, const double* db3, double* out0, double* out1) {
  if (L == 1 && Lout < 0) PB3_CASE(L1_T)
  if (L == 1 && Lout == 1) PB3_CASE(L1_A)
  if (L == 2 && Lout < 0) PB3_CASE(L2_T)
  if (L == 2 && Lout == 1) PB3_CASE(L2_N1)
  if (L == 2 && Lout == 2) PB3_CASE(L2_A)
  if (L == 3 && Lout < 0) PB3_CASE(L3_T)
  if (L == 3 && Lout == 1) PB3_CASE(L3_N1)
  if (L == 3 && Lout == 2) PB3_CASE(L3_N2)
  if (L == 3 && Lout == 3) PB3_CASE(L3_A)
  return -1;
}

void h_sh(int L, const double* n, double* Y) {
  if (L == 1) { double y[4]; sh_eval<double, 1>(n[0], n[1], n[2], y); memcpy(Y, y, sizeof y); }
  if (L == 2) { double y[9]; sh_eval<double, 2>(n[0], n[1], n[2], y); memcpy(Y, y, sizeof y); }
  if (L == 3) { double y[16]; sh_eval<double, 3>(n[0], n[1], n[2], y); memcpy(Y, y, sizeof y); }
}

void h_sh_grad(int L, const double* n, const double* dY, double* dn) {
  double g[3];
  if (L == 1) { double y[4]; memcpy(y, dY, sizeof y); sh_grad<double, 1>(n[0], n[1], n[2], y, g); }
  if (L == 2) { double y[9]; memcpy(y, dY, sizeof y); sh_grad<double, 2>(n[0], n[1], n[2], y, g); }
  if (L == 3) { double y[16]; memcpy(y, dY, sizeof y); sh_grad<double, 3>(n[0], n[1], n[2], y, g); }
  memcpy(dn, g, sizeof g);
}

// env_after_mlp != 0: b / db without the envelope, which is returned separately in env[0], env[1] (value, derivative)
void h_radial2(double d, double rc, int p, int env_after_mlp, double* b, double* db, double* env) {
  double bb[kNumBessel], dd[kNumBessel];
  RadialParams<double> rp;
  for (int n = 0; n < kNumBessel; ++n) rp.w[n] = (n + 1) * 3.14159265358979323846 / rc;
  rp.pref = std::sqrt(2.0 / rc); rp.rc = rc; rp.p = p; rp.env_after_mlp = env_after_mlp;
  radial_eval<double>(d, rp, bb, dd);
  memcpy(b, bb, sizeof bb); memcpy(db, dd, sizeof dd);
  envelope_eval<double>(d, rp, env[0], env[1]);
}

void h_radial(double d, double rc, int p, double* b, double* db) {
  double bb[kNumBessel], dd[kNumBessel];
  RadialParams<double> rp;
  rp.env_after_mlp = 0;
  for (int n = 0; n < kNumBessel; ++n) rp.w[n] = (n + 1) * 3.14159265358979323846 / rc;
  rp.pref = std::sqrt(2.0 / rc); rp.rc = rc; rp.p = p;
  radial_eval<double>(d, rp, bb, dd);
  memcpy(b, bb, sizeof bb); memcpy(db, dd, sizeof dd);
}

void h_mlp(const double* b, const double* A0, const double* A1, const double* A2, const double* A1t,
           const double* A2t, const double* dh3, double* h3, double* db) {
  double bb[kNumBessel], hh[kHidden], dh[kHidden], dbb[kNumBessel];
  alignas(16) double zs[3 * kHidden];
  memcpy(bb, b, sizeof bb); memcpy(dh, dh3, sizeof dh);
  (void)A1; (void)A2;
  mlp_hidden_fwd<double>(bb, A0, A1, A2, hh, zs, 1);
  mlp_hidden_bwd<double>(zs, 1, A0, A1t, A2t, dh, dbb);
  memcpy(h3, hh, sizeof hh); memcpy(db, dbb, sizeof dbb);
}

void h_edge_grad(const double* v, double dd, const double* dn, double* g) {
  double vv[3] = {v[0], v[1], v[2]}, dnn[3] = {dn[0], dn[1], dn[2]}, gg[3];
  const double d0 = std::sqrt(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
  edge_vector_grad<double>(vv, d0, d0 + 1e-9, dd, dnn, gg);
  memcpy(g, gg, sizeof gg);
}
}
