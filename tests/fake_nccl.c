/* A stand-in for the communication library whose calls fail: lets the CPU tests check that
 * the C ABI reports TCEC_ERR_COMM instead of crashing or blocking when NCCL does not work. */
#include <stddef.h>
typedef struct { char internal[128]; } ncclUniqueId;
int ncclGetUniqueId(ncclUniqueId* id) { (void)id; return 2; /* ncclSystemError */ }
int ncclCommInitRankConfig(void** comm, int n, ncclUniqueId id, int rank, void* cfg) {
  (void)comm; (void)n; (void)id; (void)rank; (void)cfg; return 2;
}
int ncclCommDestroy(void* comm) { (void)comm; return 0; }
int ncclBroadcast(const void* s, void* r, size_t c, int t, int root, void* comm, void* stream) {
  (void)s; (void)r; (void)c; (void)t; (void)root; (void)comm; (void)stream; return 2;
}
int ncclGroupStart(void) { return 0; }
int ncclGroupEnd(void) { return 0; }
