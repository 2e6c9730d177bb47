/* A plain C consumer of the C ABI: no Python, no torch.  Builds a small GQA decoding problem with
 * cudaMalloc / cudaMemcpy, calls b200attn_decode_fwd and b200attn_paged_decode_fwd through
 * include/b200attn.h, and checks both against a double-precision loop on the host.
 * Exit code 0 and the line "c-abi consumer ok" on success. */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "b200attn.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
  fprintf(stderr, "%s:%d cuda error %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); return 2; } } while (0)

/* bf16 <-> float on the host (round to nearest even) */
static uint16_t f2bf(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float bf2f(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
static float frand(uint32_t* s) { *s = *s * 1664525u + 1013904223u; return ((*s >> 8) & 0xffff) / 32768.0f - 1.0f; }

enum { B = 3, HQ = 8, HKV = 2, D = 128, CAP = 640, PAGE = 64 };

int main(void) {
  const int lens[B] = {640, 1, 333};
  const size_t nq = (size_t)B * HQ * D, nkv = (size_t)B * CAP * HKV * D;
  uint16_t *hq = malloc(nq * 2), *hk = malloc(nkv * 2), *hv = malloc(nkv * 2), *ho = malloc(nq * 2), *ho2 = malloc(nq * 2);
  uint32_t seed = 12345u;
  for (size_t i = 0; i < nq; ++i) hq[i] = f2bf(frand(&seed));
  for (size_t i = 0; i < nkv; ++i) { hk[i] = f2bf(frand(&seed)); hv[i] = f2bf(frand(&seed)); }

  void *dq, *dk, *dv, *dout, *dws; int32_t* dlens;
  CHECK_CUDA(cudaMalloc(&dq, nq * 2)); CHECK_CUDA(cudaMalloc(&dk, nkv * 2)); CHECK_CUDA(cudaMalloc(&dv, nkv * 2));
  CHECK_CUDA(cudaMalloc(&dout, nq * 2)); CHECK_CUDA(cudaMalloc((void**)&dlens, sizeof(lens)));
  CHECK_CUDA(cudaMemcpy(dq, hq, nq * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dk, hk, nkv * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dv, hv, nkv * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dlens, lens, sizeof(lens), cudaMemcpyHostToDevice));

  b200attn_decode_args a;
  memset(&a, 0, sizeof(a));
  a.q = dq; a.k_cache = dk; a.v_cache = dv; a.o = dout;
  a.dtype = B200ATTN_BF16; a.batch = B; a.heads_q = HQ; a.heads_kv = HKV; a.head_dim = D;
  a.max_seqlen = CAP; a.seqlens = dlens;
  a.q_stride_b = HQ * D; a.q_stride_h = D;
  a.k_stride_b = (int64_t)CAP * HKV * D; a.k_stride_t = HKV * D; a.k_stride_h = D;
  a.v_stride_b = a.k_stride_b; a.v_stride_t = a.k_stride_t; a.v_stride_h = a.k_stride_h;
  a.o_stride_b = HQ * D; a.o_stride_h = D;
  a.softmax_scale = 1.0f / sqrtf((float)D);
  a.workspace_bytes = b200attn_decode_workspace_bytes(&a);
  CHECK_CUDA(cudaMalloc(&dws, a.workspace_bytes));
  a.workspace = dws;
  if (b200attn_abi_version() != B200ATTN_ABI_VERSION) { fprintf(stderr, "abi version\n"); return 3; }
  int rc = b200attn_decode_fwd(&a, 0);
  if (rc != B200ATTN_OK) { fprintf(stderr, "decode_fwd: %s\n", b200attn_strerror(rc)); return 4; }
  CHECK_CUDA(cudaDeviceSynchronize());
  CHECK_CUDA(cudaMemcpy(ho, dout, nq * 2, cudaMemcpyDeviceToHost));

  /* the same keys as a page pool: sequence b's page i lives at pool page (B - 1 - b) * pages + i */
  const int pages = CAP / PAGE;
  int32_t table[B][CAP / PAGE];
  void *dkp, *dvp; int32_t* dtable;
  CHECK_CUDA(cudaMalloc(&dkp, nkv * 2)); CHECK_CUDA(cudaMalloc(&dvp, nkv * 2));
  CHECK_CUDA(cudaMalloc((void**)&dtable, sizeof(table)));
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < pages; ++i) {
      table[b][i] = (B - 1 - b) * pages + i;
      const size_t page_elems = (size_t)PAGE * HKV * D;
      CHECK_CUDA(cudaMemcpy((uint16_t*)dkp + table[b][i] * page_elems, hk + ((size_t)b * CAP + (size_t)i * PAGE) * HKV * D,
                            page_elems * 2, cudaMemcpyHostToDevice));
      CHECK_CUDA(cudaMemcpy((uint16_t*)dvp + table[b][i] * page_elems, hv + ((size_t)b * CAP + (size_t)i * PAGE) * HKV * D,
                            page_elems * 2, cudaMemcpyHostToDevice));
    }
  CHECK_CUDA(cudaMemcpy(dtable, table, sizeof(table), cudaMemcpyHostToDevice));
  b200attn_paged_decode_args g;
  memset(&g, 0, sizeof(g));
  g.q = dq; g.k_pages = dkp; g.v_pages = dvp; g.o = dout;
  g.dtype = B200ATTN_BF16; g.batch = B; g.heads_q = HQ; g.heads_kv = HKV; g.head_dim = D;
  g.page_size = PAGE; g.num_pages = B * pages; g.max_pages_per_seq = pages; g.max_seqlen = CAP;
  g.page_table = dtable; g.seqlens = dlens;
  g.q_stride_b = HQ * D; g.q_stride_h = D;
  g.k_stride_page = (int64_t)PAGE * HKV * D; g.k_stride_t = HKV * D; g.k_stride_h = D;
  g.v_stride_page = g.k_stride_page; g.v_stride_t = g.k_stride_t; g.v_stride_h = g.k_stride_h;
  g.o_stride_b = HQ * D; g.o_stride_h = D;
  g.softmax_scale = a.softmax_scale;
  g.workspace = dws; g.workspace_bytes = a.workspace_bytes;
  if (b200attn_paged_decode_workspace_bytes(&g) > a.workspace_bytes) { fprintf(stderr, "paged workspace\n"); return 5; }
  rc = b200attn_paged_decode_fwd(&g, 0);
  if (rc != B200ATTN_OK) { fprintf(stderr, "paged_decode_fwd: %s\n", b200attn_strerror(rc)); return 6; }
  CHECK_CUDA(cudaDeviceSynchronize());
  CHECK_CUDA(cudaMemcpy(ho2, dout, nq * 2, cudaMemcpyDeviceToHost));

  /* host reference in double precision from the same rounded inputs */
  double max_err = 0.0;
  static double s[CAP];
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < HQ; ++h) {
      const int hk_ = h / (HQ / HKV), n = lens[b];
      double m = -1e300, l = 0.0, o[D];
      for (int t = 0; t < n; ++t) {
        double acc = 0.0;
        for (int d = 0; d < D; ++d)
          acc += (double)bf2f(hq[((size_t)b * HQ + h) * D + d]) * bf2f(hk[(((size_t)b * CAP + t) * HKV + hk_) * D + d]);
        s[t] = acc * a.softmax_scale;
        if (s[t] > m) m = s[t];
      }
      for (int d = 0; d < D; ++d) o[d] = 0.0;
      for (int t = 0; t < n; ++t) {
        const double p = exp(s[t] - m);
        l += p;
        for (int d = 0; d < D; ++d) o[d] += p * bf2f(hv[(((size_t)b * CAP + t) * HKV + hk_) * D + d]);
      }
      for (int d = 0; d < D; ++d) {
        const double ref = n > 0 ? o[d] / l : 0.0;
        const size_t idx = ((size_t)b * HQ + h) * D + d;
        const double e1 = fabs(ref - bf2f(ho[idx]));
        if (e1 > max_err) max_err = e1;
        if (ho[idx] != ho2[idx]) { fprintf(stderr, "paged result differs from padded at %zu\n", idx); return 7; }
      }
    }
  printf("max abs error vs double-precision host loop: %.5f\n", max_err);
  if (!(max_err <= 2e-2)) return 8;
  /* argument errors come back as codes, nothing is thrown */
  a.head_dim = 100;
  if (b200attn_decode_fwd(&a, 0) != B200ATTN_ERR_HEAD_DIM) return 9;
  printf("c-abi consumer ok\n");
  return 0;
}
