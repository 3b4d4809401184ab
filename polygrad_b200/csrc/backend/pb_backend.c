/*
 * pb_backend.c -- the two IR-facing entry points of the CUDA backend row.
 *
 * exec_plan.c's cuda_lower_item (reference: src/exec_plan.c:529-582) calls
 *   poly_linearize_cuda(ctx, scheduled_root, &n)  -> PolyUOp* array (caller frees)
 *   poly_render_cuda(array, n, fn_name, block)    -> C string (caller frees)
 *   poly_compile_cuda(string, fn_name)            -> PolyCudaProgram*
 * in that order.  The reference versions (src/render_cuda.c:176, :196) run the
 * whole rewrite pipeline and print scalar CUDA C.  Here the "linearized" array
 * is the scheduled SINK itself after one symbolic simplification -- the form in
 * which every reduction is still one REDUCE node -- and the renderer analyses
 * that tree: it either names a precompiled sm_100a kernel with its arguments
 * (header-only text) or emits CUDA C built around the same tree.  Either text
 * starts with "//PB200" lines that poly_compile_cuda understands.
 *
 * cuda_lower_item scans the array for SPECIAL ops to size the grid; there are
 * none, so it passes grid 1 / block 256, which poly_cuda_launch ignores: every
 * program carries its own launch geometry.
 */
#include "pb_kern.h"
#include "pat.h"
#include "codegen.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

PolyUOp **poly_linearize_cuda(PolyCtx *ctx, PolyUOp *sink, int *n_out) {
  if (!ctx || !sink || !n_out) return NULL;
  sink = poly_graph_rewrite(ctx, sink, poly_symbolic_simple());
  if (!sink) { fprintf(stderr, "polygrad: cuda: symbolic rewrite failed\n"); return NULL; }
  PolyUOp **arr = malloc(sizeof(PolyUOp *));
  if (!arr) return NULL;
  arr[0] = sink;
  *n_out = 1;
  return arr;
}

char *poly_render_cuda(PolyUOp **uops, int n, const char *fn_name, int launch_bounds) {
  (void)launch_bounds;
  if (!uops || n != 1 || !uops[0] || uops[0]->op != POLY_OP_SINK) {
    fprintf(stderr, "polygrad: cuda: poly_render_cuda expects the array returned by poly_linearize_cuda\n");
    return NULL;
  }
  PbKern k;
  if (pb_kern_build(&k, uops[0]) != 0) {
    fprintf(stderr, "polygrad: cuda: cannot lower kernel %s: %s\n", fn_name ? fn_name : "?", k.err);
    pb_kern_free(&k);
    return NULL;
  }
  if (getenv("POLY_B200_DUMP_UOPS")) {      /* the analysed tree, sources first: index, node, indices of its sources */
    fprintf(stderr, "=== UOPS %s ===\n", fn_name ? fn_name : "?");
    for (int i = 0; i < k.n_nodes; i++) {
      char *t = poly_uop_str(k.nodes[i].u);
      fprintf(stderr, "%4d %s <-", i, t ? t : "?");
      for (int j = 0; j < k.nodes[i].u->n_src; j++) fprintf(stderr, " %d", pb_kern_node(&k, k.nodes[i].u->src[j]));
      fprintf(stderr, "\n");
      free(t);
    }
    fprintf(stderr, "=== END UOPS ===\n");
  }
  char *src = NULL;
  const char *no_aot = getenv("POLY_B200_NO_AOT");
  if (!no_aot || no_aot[0] == '0') src = pb_classify_aot(&k, fn_name);
  if (!src) src = pb_render_jit(&k, fn_name);
  if (!src) fprintf(stderr, "polygrad: cuda: cannot lower kernel %s: %s\n", fn_name ? fn_name : "?", k.err);
  pb_kern_free(&k);
  return src;
}
