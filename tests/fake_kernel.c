/* A host-only stand-in for a compiled kernel library, for testing the host runtime without a
 * device: it exports the four per-kernel symbols for a kernel named "probe" with two tensors
 * (x: [N, 4] f32 read, y: [{"mul":["N",2]}] i32 write), one runtime parameter N, and a workspace
 * of 96 * N bytes rounded up to 512. launch_probe records its arguments instead of launching. */
#include <stdint.h>
#include <stddef.h>

static int64_t record[8];
static int64_t launches;

int kernel_config_probe(int64_t* cfg) {
  if (!cfg) return -1;
  cfg[0] = 2; cfg[1] = 1; cfg[2] = 1; cfg[3] = 0; cfg[4] = 0;
  return 0;
}

const char* kernel_metadata_probe(void) {
  return "{\"version\":1,\"name\":\"probe\",\"target\":\"sm_100a\",\"kind\":\"mixed\",\"groups\":1,"
         "\"disjoint_external\":true,\"device_resources\":null,\"tensors\":["
         "{\"name\":\"x\",\"dtype\":\"f32\",\"shape\":[\"N\",4],\"layout\":\"linear\",\"access\":\"read\"},"
         "{\"name\":\"y\",\"dtype\":\"i32\",\"shape\":[{\"mul\":[\"N\",2]}],\"layout\":\"linear\",\"access\":\"write\"}],"
         "\"parameters\":[{\"name\":\"N\",\"minimum\":2,\"multiple\":2}],\"workspace\":true}";
}

int workspace_size_probe(uint64_t* bytes, int64_t n) {
  if (!bytes) return -1;
  *bytes = 0;
  if (n < 0) return -1;
  if ((uint64_t)n > (uint64_t)INT64_MAX / 96u) return -1;
  *bytes = ((uint64_t)n * 96u + 511u) / 512u * 512u;
  return 0;
}

int launch_probe(void* stream, void* x, void* y, void* workspace, int64_t n) {
  record[0] = (int64_t)(intptr_t)stream;
  record[1] = (int64_t)(intptr_t)x;
  record[2] = (int64_t)(intptr_t)y;
  record[3] = (int64_t)(intptr_t)workspace;
  record[4] = n;
  launches += 1;
  return n == 666 ? 7 : 0;
}

int64_t probe_launches(void) { return launches; }
void probe_last_call(int64_t* out) { for (int i = 0; i < 5; ++i) out[i] = record[i]; }
