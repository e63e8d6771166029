/* A gather of an escape-time image over N ranks driven through include/vrhi.h only: plain C, one
 * process per GPU (fork), the library's one bootstrap need (an all-gather of small records) served
 * from a shared anonymous mapping.  Three steps run back to back with a different Julia constant each
 * and no barrier between them; every step's gathered image must equal, bit for bit, the image the
 * same rank computes alone.  Also sums a small float array over the ranks.
 *
 *   group_gather_test [ranks]        exit 0 = pass, 77 = fewer GPUs than ranks, anything else = fail
 */
#define _GNU_SOURCE
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include "vrhi.h"

enum { W = 1024, H = 1024, CHUNK = 16, STEPS = 3, GROUPS = 2, MAXR = 8, REC = 256 };

typedef struct {
  volatile int arrived[2];  /* sense-reversing barrier */
  volatile int sense;
  unsigned char records[MAXR][REC];
} shared_t;

typedef struct { shared_t *sh; int world, rank, local_sense; } boot_t;

static void barrier(boot_t *b) {
  b->local_sense ^= 1;
  if (__sync_add_and_fetch(&b->sh->arrived[b->local_sense], 1) == b->world) {
    b->sh->arrived[b->local_sense] = 0;
    __sync_synchronize();
    b->sh->sense = b->local_sense;
  } else {
    int spins = 0;
    while (b->sh->sense != b->local_sense) {
      usleep(100);
      if (++spins > 300000) { fprintf(stderr, "rank %d: barrier timed out\n", b->rank); _exit(3); }
    }
  }
}

static int allgather(void *user, const void *send, void *recv, uint64_t bytes) {
  boot_t *b = (boot_t *)user;
  if (bytes > REC) return 1;
  memcpy(b->sh->records[b->rank], send, bytes);
  __sync_synchronize();
  barrier(b);
  for (int r = 0; r < b->world; ++r) memcpy((char *)recv + (size_t)r * bytes, b->sh->records[r], bytes);
  barrier(b);
  return 0;
}

#define OK(call)                                                                               \
  do {                                                                                         \
    int rc__ = (call);                                                                         \
    if (rc__ != VRHI_OK) {                                                                     \
      fprintf(stderr, "rank %d: %s -> %d (%s)\n", rank, #call, rc__, vrhi_last_error());       \
      return 1;                                                                                \
    }                                                                                          \
  } while (0)

static void julia(vrhi_escape_params *p, float ci) {
  memset(p, 0, sizeof *p);
  p->size = sizeof *p;
  p->kind = VRHI_ESCAPE_JULIA; p->mode = VRHI_ESCAPE_EXACT; p->test = VRHI_TEST_NORM2_GT; p->output = VRHI_OUT_COUNT_U32;
  p->width = W; p->height = H; p->max_iter = 1000;
  p->x0 = -1.6f; p->y0 = -1.6f; p->dx = 3.2f / W; p->dy = 3.2f / H;
  p->cr = -0.8f; p->ci = ci; p->bound = 4.0f;
}

static int run_rank(shared_t *sh, int world, int rank) {
  boot_t boot = {sh, world, rank, 0};
  vrhi_device dev; vrhi_stream st; vrhi_group grp; vrhi_exchange ex;
  vrhi_buffer image, ref, vec;
  int op;
  OK(vrhi_device_create(rank, &dev));
  OK(vrhi_stream_create(dev, &st));
  OK(vrhi_group_create(dev, (uint32_t)world, (uint32_t)rank, allgather, &boot, &grp));
  OK(vrhi_buffer_create(dev, (uint64_t)W * H * 4, VRHI_IMAGE, &image));
  OK(vrhi_buffer_create(dev, (uint64_t)W * H * 4, VRHI_IMAGE, &ref));
  OK(vrhi_buffer_fill_u8(image, 0, 0xff, (uint64_t)W * H * 4, st));
  OK(vrhi_exchange_create(grp, image, W, H, CHUNK, &ex));
  OK(vrhi_op_lookup("escape_time", &op));
  vrhi_row_partition part;
  OK(vrhi_partition_rows(H, CHUNK, (uint32_t)world, (uint32_t)rank, VRHI_PART_CYCLIC, &part));
  uint32_t *got[STEPS], *want = NULL;
  for (int s = 0; s < STEPS; ++s) OK(vrhi_host_alloc((uint64_t)W * H * 4, (void **)&got[s]));
  OK(vrhi_host_alloc((uint64_t)W * H * 4, (void **)&want));

  const float ci[STEPS] = {0.156f, 0.2f, -0.11f};
  for (int s = 0; s < STEPS; ++s) {  /* no host synchronisation and no barrier inside this loop */
    vrhi_buffer wire, bytes;
    OK(vrhi_exchange_planes(ex, &wire, &bytes));  /* bytes == NULL where the exchange does not squeeze the counts */
    for (int g = 0; g < GROUPS; ++g) {
      vrhi_escape_params p;
      julia(&p, ci[s]);
      const uint32_t count = (part.chunk_count - g + GROUPS - 1) / GROUPS;  /* slabs g, g+GROUPS, ... */
      p.chunk_rows = part.chunk_rows; p.chunk_first = part.chunk_first + g * part.chunk_step;
      p.chunk_step = part.chunk_step * GROUPS; p.chunk_count = count;
      vrhi_arg args[3] = {{image, 0, 0, VRHI_IMAGE, 0}, {wire, 0, 0, VRHI_IMAGE, 0}, {bytes, 0, 0, VRHI_IMAGE, 0}};
      OK(vrhi_op_launch(st, op, args, bytes ? 3 : 2, &p, sizeof p));
      OK(vrhi_exchange_publish(ex, st, (uint32_t)g, count, GROUPS));
    }
    OK(vrhi_exchange_complete(ex, st));
    OK(vrhi_buffer_download(image, 0, got[s], (uint64_t)W * H * 4, st));
  }
  OK(vrhi_stream_synchronize(st));
  OK(vrhi_exchange_check(ex));

  int bad = 0;
  for (int s = 0; s < STEPS; ++s) {  /* the same image computed by this rank alone */
    vrhi_escape_params p;
    julia(&p, ci[s]);
    vrhi_arg a = {ref, 0, 0, VRHI_IMAGE, 0};
    OK(vrhi_op_launch(st, op, &a, 1, &p, sizeof p));
    OK(vrhi_buffer_download(ref, 0, want, (uint64_t)W * H * 4, st));
    OK(vrhi_stream_synchronize(st));
    uint64_t sum = 0;
    size_t diff = 0;
    for (size_t k = 0; k < (size_t)W * H; ++k) { diff += got[s][k] != want[k]; sum += want[k]; }
    if (diff || sum == 0) { fprintf(stderr, "rank %d step %d: %zu pixels differ (sum of counts %llu)\n", rank, s, diff, (unsigned long long)sum); bad = 1; }
  }

  /* sum of a small array over the ranks: element k of rank r is k + r/8, twice in a row */
  enum { NV = 4100 };
  float hv[NV];
  OK(vrhi_buffer_create(dev, NV * 4, VRHI_STORAGE_BUFFER, &vec));
  for (int round = 0; round < 2; ++round) {
    for (int k = 0; k < NV; ++k) hv[k] = (float)(k + round) + (float)rank / 8.0f;
    OK(vrhi_buffer_upload(vec, 0, hv, NV * 4, st));
    OK(vrhi_group_all_reduce_sum_f32(grp, vec, 0, NV, st));
    OK(vrhi_buffer_download(vec, 0, hv, NV * 4, st));
    OK(vrhi_stream_check(st));
    for (int k = 0; k < NV; ++k) {
      float w = 0.f;
      for (int r = 0; r < world; ++r) w += (float)(k + round) + (float)r / 8.0f;  /* rank order, as the library adds */
      if (hv[k] != w) { fprintf(stderr, "rank %d: all-reduce element %d is %g, expected %g\n", rank, k, hv[k], w); bad = 1; break; }
    }
  }

  barrier(&boot);  /* nobody tears down while a peer may still store into its memory */
  OK(vrhi_exchange_destroy(ex));
  OK(vrhi_group_destroy(grp));
  for (int s = 0; s < STEPS; ++s) vrhi_host_free(got[s]);
  vrhi_host_free(want);
  vrhi_buffer_destroy(vec); vrhi_buffer_destroy(ref); vrhi_buffer_destroy(image);
  vrhi_stream_destroy(st); vrhi_device_destroy(dev);
  if (!bad) printf("rank %d of %d: %d steps gathered bit-exact, all-reduce exact\n", rank, world, STEPS);
  return bad;
}

int main(int argc, char **argv) {
  int world = argc > 1 ? atoi(argv[1]) : 2;
  if (world < 1 || world > MAXR) { fprintf(stderr, "ranks: 1..%d\n", MAXR); return 2; }
  shared_t *sh = mmap(NULL, sizeof *sh, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  if (sh == MAP_FAILED) { perror("mmap"); return 2; }
  memset((void *)sh, 0, sizeof *sh);
  pid_t kids[MAXR];
  for (int r = 0; r < world; ++r) {  /* no CUDA call before the fork: every rank opens its own context */
    kids[r] = fork();
    if (kids[r] < 0) { perror("fork"); return 2; }
    if (kids[r] == 0) {
      int n = 0;
      if (vrhi_device_count(&n) != VRHI_OK || n < world) _exit(77);
      int code = run_rank(sh, world, r);
      fflush(NULL);  /* _exit does not flush stdio */
      _exit(code);
    }
  }
  int worst = 0;
  for (int r = 0; r < world; ++r) {
    int status = 0;
    waitpid(kids[r], &status, 0);
    int code = WIFEXITED(status) ? WEXITSTATUS(status) : 99;
    if (code != 0 && (worst == 0 || worst == 77)) worst = code;
  }
  return worst;
}
