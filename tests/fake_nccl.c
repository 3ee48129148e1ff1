/* A stand-in for libnccl used by the failure-handling test: collectives do nothing, and the asynchronous error state the
 * library polls (ncclCommGetAsyncError) is whatever the test set.  Built by the test with gcc; never shipped. */
#include <stddef.h>
#include <string.h>
typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fake_comm { int rank, world, aborted, destroyed; } fake_comm;
static fake_comm g_comm;
static int g_async_error = 0, g_aborts = 0, g_allreduces = 0;
void fake_nccl_set_async_error(int code) { g_async_error = code; }
int fake_nccl_abort_count(void) { return g_aborts; }
int fake_nccl_allreduce_count(void) { return g_allreduces; }
int ncclGetUniqueId(ncclUniqueId *id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(fake_comm **comm, int world, ncclUniqueId id, int rank) { (void)id; g_comm.rank = rank; g_comm.world = world; *comm = &g_comm; return 0; }
int ncclAllReduce(const void *s, void *r, size_t n, int dt, int op, fake_comm *c, void *stream) { (void)s; (void)r; (void)n; (void)dt; (void)op; (void)c; (void)stream; ++g_allreduces; return 0; }
int ncclCommDestroy(fake_comm *c) { c->destroyed = 1; return 0; }
int ncclCommAbort(fake_comm *c) { c->aborted = 1; ++g_aborts; return 0; }
int ncclCommGetAsyncError(fake_comm *c, int *err) { (void)c; *err = g_async_error; return 0; }
const char *ncclGetErrorString(int code) { return code == 6 ? "remote process exited or there was a network error" : code == 0 ? "no error" : "fake error"; }
