/* Minimal C host of the contracts C ABI: opens the CPU bundle and prints the runtime catalog.
 *   gcc -o c_host examples/c_host.c -Iinference_b200/csrc/include -Linference_b200/_native -lswb200_capi \
 *       -Wl,-rpath,$PWD/inference_b200/_native
 *   PYTHONPATH=<site-packages with torch> ./c_host $PWD
 */
#include <stdio.h>
#include "swb200_contracts.h"
int main(int argc, char** argv) {
  swb_runtime* rt = 0;
  int rc = swb_rt_open("cpu", argc > 1 ? argv[1] : 0, &rt);
  if (rc) { printf("open failed %d: %s\n", rc, swb_rt_last_error()); return 1; }
  char* js = 0;
  rc = swb_rt_catalog_json(rt, &js);
  printf("rc=%d %s\n", rc, js ? js : "(null)");
  swb_rt_free_string(js);
  swb_rt_close(rt);
  return rc;
}
