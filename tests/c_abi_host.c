/* A C (not C++) host of the C ABI: includes the public header, loads the library at run time and
 * walks the calls a foreign-language binding makes first.  Built and run by tests/test_c_abi.py with gcc. */
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "pypto_b200.h"

typedef const char* (*str_fn)(void);
typedef int (*create_fn)(int, pto_worker**);
typedef int (*destroy_fn)(pto_worker*);

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  void* lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
  if (!lib) { fprintf(stderr, "dlopen: %s\n", dlerror()); return 3; }
  str_fn version = (str_fn)dlsym(lib, "pto_version");
  str_fn last_error = (str_fn)dlsym(lib, "pto_last_error");
  str_fn op_list = (str_fn)dlsym(lib, "pto_op_list");
  create_fn create = (create_fn)dlsym(lib, "pto_worker_create");
  destroy_fn destroy = (destroy_fn)dlsym(lib, "pto_worker_destroy");
  if (!version || !last_error || !op_list || !create || !destroy) return 4;
  printf("version=%s\n", version());
  int n = 0;
  for (const char* p = op_list(); *p; p += strlen(p) + 1) { printf("op=%s\n", p); ++n; }
  if (n == 0) return 5;
  if (sizeof(pto_chip_tensor) != 48) return 6;     /* layout relied on by device code */
  pto_worker* w = NULL;
  int st = create(0, &w);
  printf("worker_create=%d%s%s\n", st, st ? " error=" : "", st ? last_error() : "");
  if (st == PTO_OK) {
    if (destroy(w) != PTO_OK) return 7;
  } else if (last_error()[0] == 0) {
    return 8;                                        /* a failure must leave a message */
  }
  if (destroy(NULL) != PTO_OK) return 9;            /* idempotent on NULL */
  return 0;
}
