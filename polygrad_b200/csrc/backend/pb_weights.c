/*
 * pb_weights.c -- safetensors weights into an instance wherever it lives.
 *
 * poly_instance_import_weights (reference: src/instance.c:522-550) copies each
 * tensor into the instance's host array and accepts float32 files only; after
 * poly_instance_set_device(CUDA) the device buffers, which are what the plans
 * read, keep their old contents.  poly_b200_instance_import_weights decodes with
 * polygrad's multi-dtype decoder (F32, BF16, F16; files above 2 GB,
 * src/safetensors.h:78), and puts every tensor where the instance's buffer is:
 * float32 data goes from the file bytes to the device in one copy (no host
 * array in between), 16-bit data is widened on the host first; buffers still in
 * host memory are filled in place.  Tensors are matched by name, as in the
 * reference; unknown names are reported and skipped, a size mismatch is an
 * error.
 */
#include "instance.h"
#include "safetensors.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int poly_b200_instance_import_weights(PolyInstance *inst, const unsigned char *data, long long len, long long *bytes_to_device);

static int find_buf(PolyInstance *inst, const char *name) {
  int n = poly_instance_buf_count(inst);
  for (int i = 0; i < n; i++) {
    const char *b = poly_instance_buf_name(inst, i);
    if (b && strcmp(b, name) == 0) return i;
  }
  return -1;
}

int poly_b200_instance_import_weights(PolyInstance *inst, const unsigned char *data, long long len, long long *bytes_to_device) {
  if (bytes_to_device) *bytes_to_device = 0;
  if (!inst || !data || len <= 0) return -1;
  int n_views = 0;
  char *metadata = NULL;
  PolySafetensorViewEx *views = poly_safetensors_decode_ex(data, (int64_t)len, &n_views, &metadata);
  if (!views) { fprintf(stderr, "polygrad: cuda: import_weights: not a safetensors file\n"); return -1; }
  int rc = 0;
  for (int i = 0; i < n_views; i++) {
    const PolySafetensorViewEx *v = &views[i];
    int bi = rc == 0 ? find_buf(inst, v->name) : -1;
    if (rc != 0) { free(v->name); continue; }
    if (bi < 0) {
      fprintf(stderr, "poly_b200_instance_import_weights: unknown tensor '%s'\n", v->name);
      free(v->name);
      continue;
    }
    int64_t shape[8], numel = 1, host_numel = 0;
    int nd = poly_instance_buf_shape(inst, bi, shape, 8);
    for (int d = 0; d < nd; d++) numel *= shape[d];
    if (numel != v->numel) {
      fprintf(stderr, "polygrad: cuda: import_weights: '%s' has %lld elements, the instance expects %lld\n", v->name,
              (long long)v->numel, (long long)numel);
      rc = -1; free(v->name); continue;
    }
    const float *src = NULL; float *widened = NULL;
    if (v->dtype == POLY_ST_F32) src = (const float *)v->raw_data;
    else if (v->dtype == POLY_ST_BF16 || v->dtype == POLY_ST_F16) src = widened = poly_safetensors_to_f32(v);
    if (!src) {
      fprintf(stderr, "polygrad: cuda: import_weights: '%s' has a dtype that float32 buffers cannot take\n", v->name);
      rc = -1; free(v->name); continue;
    }
    const size_t bytes = (size_t)numel * sizeof(float);
    float *host = poly_instance_buf_data(inst, bi, &host_numel);     /* NULL when device-resident (src/instance.h:75-78) */
    if (host) memcpy(host, src, bytes);
    else if (poly_instance_upload_buf(inst, bi, src, bytes) != 0) {
      fprintf(stderr, "polygrad: cuda: import_weights: upload of '%s' failed\n", v->name);
      rc = -1;
    } else if (bytes_to_device) *bytes_to_device += (long long)bytes;
    free(widened);
    free(v->name);
  }
  free(views);
  free(metadata);
  return rc;
}
