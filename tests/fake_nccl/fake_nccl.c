/* Stand-in for libnccl.so.2 used by the failure-path tests (loaded through FITRE_NCCL_LIBRARY).
 * It moves no data.  Environment variables choose how it misbehaves:
 *   FAKE_NCCL_INIT_SLEEP        seconds ncclCommInitRank sleeps before returning (a peer that never joins)
 *   FAKE_NCCL_INIT_RESULT       result code of ncclCommInitRank
 *   FAKE_NCCL_STALL_MS          every collective parks the stream in a HOST function for that long
 *                               (the GPU stays idle: nothing on the device waits or spins)
 *   FAKE_NCCL_ERROR_AFTER_POLLS ncclCommGetAsyncError reports ncclRemoteError after that many polls
 * fake_nccl_count(i) returns how often abort (0), destroy (1), a collective (2), a poll (3) was called. */
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

typedef struct { char internal[128]; } ncclUniqueId;
static int counts[4];

static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
}

int ncclGetUniqueId(ncclUniqueId *id) {
    memset(id, 7, sizeof *id);
    return 0;
}
int ncclCommInitRank(void **comm, int nranks, ncclUniqueId id, int rank) {
    (void)nranks; (void)id; (void)rank;
    int s = env_int("FAKE_NCCL_INIT_SLEEP", 0);
    if (s > 0) sleep((unsigned)s);
    *comm = (void *)0x10;
    return env_int("FAKE_NCCL_INIT_RESULT", 0);
}
int ncclCommDestroy(void *comm) { (void)comm; counts[1]++; return 0; }
int ncclCommAbort(void *comm) { (void)comm; counts[0]++; return 0; }
int ncclCommGetAsyncError(void *comm, int *state) {
    (void)comm;
    counts[3]++;
    int after = env_int("FAKE_NCCL_ERROR_AFTER_POLLS", -1);
    *state = (after >= 0 && counts[3] > after) ? 6 : 0;
    return 0;
}
static void CUDART_CB nap(void *ms) { usleep(1000 * (useconds_t)(long)ms); }
static int collective(cudaStream_t stream) {
    counts[2]++;
    int ms = env_int("FAKE_NCCL_STALL_MS", 0);
    if (ms > 0) cudaLaunchHostFunc(stream, nap, (void *)(long)ms);
    return 0;
}
int ncclAllReduce(const void *s, void *r, size_t n, int dt, int op, void *comm, cudaStream_t stream) {
    (void)s; (void)r; (void)n; (void)dt; (void)op; (void)comm;
    return collective(stream);
}
int ncclReduce(const void *s, void *r, size_t n, int dt, int op, int root, void *comm, cudaStream_t stream) {
    (void)s; (void)r; (void)n; (void)dt; (void)op; (void)root; (void)comm;
    return collective(stream);
}
int ncclBroadcast(const void *s, void *r, size_t n, int dt, int root, void *comm, cudaStream_t stream) {
    (void)s; (void)r; (void)n; (void)dt; (void)root; (void)comm; (void)stream;
    return 0;   /* set-up traffic: never stalled */
}
int ncclAllGather(const void *s, void *r, size_t n, int dt, void *comm, cudaStream_t stream) {
    (void)s; (void)r; (void)n; (void)dt; (void)comm; (void)stream;
    return 0;   /* set-up traffic: the gathered IPC handles stay zero, so the peer path stays off */
}
const char *ncclGetErrorString(int r) { return r == 6 ? "remote error (fake)" : "fake result"; }
int fake_nccl_count(int which) { return counts[which & 3]; }
