/* A plain-C consumer of the library: proves that include/fmms_b200.h is valid C and that the
 * host-only entry points can be called without a GPU.  Built and run by tests/test_host_logic.py. */
#include <stdio.h>
#include <string.h>

#include "fmms_b200.h"

int main(void) {
  int plan[8];
  size_t bytes = 0;
  if (fmms_version() < 1000) return 1;
  if (strcmp(fmms_strerror(FMMS_OK), "ok") != 0) return 2;
  if (fmms_query_workspace(151936, 4096, 64, 1, &bytes) != FMMS_OK || bytes == 0) return 3;
  /* Qwen head, 64 rows, one draw, 148 SMs with 227 KiB of shared memory: the tensor-core kernel */
  if (fmms_plan(151936, 4096, 64, 1, 0, 148, 232448, plan) != FMMS_OK) return 4;
  if (plan[0] != FMMS_PATH_MMA || plan[1] != 148) return 5;
  if (fmms_plan(151936, 4096, 1, 1, 0, 148, 232448, plan) != FMMS_OK || plan[0] != FMMS_PATH_GEMV) return 6;
  /* argument checks come before any CUDA call */
  if (fmms_sample(NULL, NULL, NULL, 0, 10, 8, 1, 1, 0ull, 0ll, 0, NULL, 0ll, NULL, NULL, NULL, NULL, 0, NULL,
                  NULL) != FMMS_ERR_BAD_ARG)
    return 7;
  if (fmms_static_max_items() < 1) return 8;
  printf("c-abi ok: workspace %lu bytes, grid %d, stages %d\n", (unsigned long)bytes, plan[1], plan[4]);
  return 0;
}
