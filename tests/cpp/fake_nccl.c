/* A stand-in for NCCL for failure tests: same entry points as the handful the library binds, no communication.
 * Collectives return at once and move nothing; ncclCommGetAsyncError starts to report a remote error after
 * FAKE_NCCL_ASYNC_ERROR_AFTER polls (never, when the variable is unset).  Test infrastructure only. */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void *ncclComm_t;
typedef void *cudaStream_t;

static int g_polls = 0, g_aborts = 0, g_destroys = 0;

int fake_nccl_polls(void) { return g_polls; }
int fake_nccl_aborts(void) { return g_aborts; }
int fake_nccl_destroys(void) { return g_destroys; }

int ncclGetUniqueId(ncclUniqueId *id) { memset(id, 7, sizeof(*id)); return 0; }
int ncclCommInitRank(ncclComm_t *comm, int nranks, ncclUniqueId id, int rank) {
    (void)nranks; (void)id; (void)rank;
    *comm = malloc(16);
    return *comm ? 0 : 2;
}
int ncclCommDestroy(ncclComm_t comm) { ++g_destroys; free(comm); return 0; }
int ncclCommAbort(ncclComm_t comm) { ++g_aborts; free(comm); return 0; }
int ncclCommGetAsyncError(ncclComm_t comm, int *async_error) {
    (void)comm;
    const char *after = getenv("FAKE_NCCL_ASYNC_ERROR_AFTER");
    ++g_polls;
    *async_error = (after && g_polls > atoi(after)) ? 6 /* ncclRemoteError */ : 0;
    return 0;
}
int ncclAllGather(const void *s, void *r, size_t n, int t, ncclComm_t c, cudaStream_t st) {
    (void)s; (void)r; (void)n; (void)t; (void)c; (void)st; return 0;
}
int ncclSend(const void *s, size_t n, int t, int peer, ncclComm_t c, cudaStream_t st) {
    (void)s; (void)n; (void)t; (void)peer; (void)c; (void)st; return 0;
}
int ncclRecv(void *r, size_t n, int t, int peer, ncclComm_t c, cudaStream_t st) {
    (void)r; (void)n; (void)t; (void)peer; (void)c; (void)st; return 0;
}
int ncclGroupStart(void) { return 0; }
int ncclGroupEnd(void) { return 0; }
