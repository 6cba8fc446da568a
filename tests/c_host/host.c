/* A compiled C host for libfortis_b200.so, standing in for the object code Flang emits for a fortisc-rewritten
 * Fortran host: it declares the entry points with FIXED argument lists, exactly as the generated gather.cu of the
 * reference does for one host (mom6_zb/gather.cu:50 `void fortis_gather(const float* H0, ...)`, :82
 * `void fortis_scatter(int a0, float* H0, ...)`), and calls them without any variadic prototype in scope.  The
 * library's entries are C variadics; this program is the proof that the two calling sequences meet.
 *
 * Built three times by tests/test_gpu_c_host.py with -DSCENARIO=1|2|3:
 *   1  k-distributed host (the MOM6 Zanna-Bolton descriptors): fortis_gather(4 arrays), fortis_model_input(),
 *      mlp_forward_batched(), fortis_scatter(k, 5 arrays) for k = 1..15.  Configuration comes from the FORTIS_*_JSON /
 *      FORTIS_MODEL environment variables, as in a run of a rewritten host.
 *   2  plane chosen by argument (no k distribution): fortis_gather(k, 2 arrays), mlp_forward_batched(),
 *      fortis_scatter(k, 1 array): the first argument is an integer by value on both entries.
 *   3  fused step: fortis_step(3 gather arrays, 3 scatter arrays).
 *
 * usage: host <dir>.  Reads <dir>/g<i>.bin and <dir>/s<i>.bin (raw arrays), writes <dir>/X.bin (the gathered model
 * input, scenarios 1 and 2) and <dir>/s<i>.out.  Exit code 0 on success. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

void mlp_forward_batched(void);
void* fortis_model_input(void);
int fortis_copy_to_host(void* dst, const void* dev, long nbytes);
int fortis_last_error(void);
const char* fortis_last_error_message(void);
void fortis_sync(void);

#if SCENARIO == 1
void fortis_gather(const float* h0, const float* h1, const float* h2, const float* h3);
void fortis_scatter(int a0, float* h0, float* h1, float* h2, float* h3, float* h4);
#define NG 4
#define NS 5
#elif SCENARIO == 2
void fortis_gather(int a0, const float* h0, const float* h1);
void fortis_scatter(int a0, float* h0);
#define NG 2
#define NS 1
#else
void fortis_step(const float* g0, const float* g1, const float* g2, float* s0, float* s1, float* s2);
#define NG 3
#define NS 3
#endif

static void* slurp(const char* dir, const char* name, long* nbytes) {
  char path[1024];
  snprintf(path, sizeof path, "%s/%s", dir, name);
  FILE* f = fopen(path, "rb");
  if (!f) { fprintf(stderr, "cannot open %s\n", path); exit(2); }
  fseek(f, 0, SEEK_END);
  *nbytes = ftell(f);
  fseek(f, 0, SEEK_SET);
  void* p = malloc(*nbytes ? *nbytes : 1);
  if (fread(p, 1, *nbytes, f) != (size_t)*nbytes) { fprintf(stderr, "short read on %s\n", path); exit(2); }
  fclose(f);
  return p;
}

static void dump(const char* dir, const char* name, const void* p, long nbytes) {
  char path[1024];
  snprintf(path, sizeof path, "%s/%s", dir, name);
  FILE* f = fopen(path, "wb");
  if (!f || fwrite(p, 1, nbytes, f) != (size_t)nbytes) { fprintf(stderr, "cannot write %s\n", path); exit(2); }
  fclose(f);
}

static void check(const char* what) {
  if (fortis_last_error()) { fprintf(stderr, "%s: %s\n", what, fortis_last_error_message()); exit(3); }
}

int main(int argc, char** argv) {
  if (argc < 2) { fprintf(stderr, "usage: host <dir> [k] [xbytes]\n"); return 2; }
  const char* dir = argv[1];
  const int k = argc > 2 ? atoi(argv[2]) : 1;
  const long xbytes = argc > 3 ? atol(argv[3]) : 0;
  (void)k; (void)xbytes;
  float* g[NG]; long gn[NG];
  float* s[NS]; long sn[NS];
  char name[64];
  for (int i = 0; i < NG; i++) { snprintf(name, sizeof name, "g%d.bin", i); g[i] = (float*)slurp(dir, name, &gn[i]); }
  for (int i = 0; i < NS; i++) { snprintf(name, sizeof name, "s%d.bin", i); s[i] = (float*)slurp(dir, name, &sn[i]); }
#if SCENARIO == 1
  fortis_gather(g[0], g[1], g[2], g[3]);
  check("fortis_gather");
#elif SCENARIO == 2
  fortis_gather(k, g[0], g[1]);
  check("fortis_gather");
#endif
#if SCENARIO != 3
  if (xbytes) {                       /* materialise and dump the gathered model input before the forward consumes it */
    void* x = malloc(xbytes);
    void* dx = fortis_model_input();
    check("fortis_model_input");
    if (fortis_copy_to_host(x, dx, xbytes) != 0) return 3;
    dump(dir, "X.bin", x, xbytes);
    free(x);
  }
  mlp_forward_batched();
  check("mlp_forward_batched");
#endif
#if SCENARIO == 1
  for (int kk = 1; kk <= k; kk++) { fortis_scatter(kk, s[0], s[1], s[2], s[3], s[4]); check("fortis_scatter"); }
#elif SCENARIO == 2
  fortis_scatter(k, s[0]);
  check("fortis_scatter");
#else
  fortis_step(g[0], g[1], g[2], s[0], s[1], s[2]);
  check("fortis_step");
  fortis_sync();
#endif
  for (int i = 0; i < NS; i++) { snprintf(name, sizeof name, "s%d.out", i); dump(dir, name, s[i], sn[i]); }
  return 0;
}
