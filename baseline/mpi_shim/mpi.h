/* Single-node stand-in for the six MPI calls the reference uses to learn rank/size and to
 * broadcast the NCCL id (src/parallel/comms.cu:17-29,43).  Rank and size come from the
 * torchrun environment (RANK, WORLD_SIZE); the broadcast goes through a file under /tmp keyed
 * by MASTER_PORT.  Header-only so that the reference sources build unchanged. */
#ifndef KH_MPI_SHIM_H
#define KH_MPI_SHIM_H
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
typedef int MPI_Comm;
typedef int MPI_Datatype;
#define MPI_COMM_WORLD 0
#define MPI_BYTE 1
#define MPI_SUCCESS 0
static int kh_mpi_env(const char *k, int d) { const char *v = getenv(k); return v ? atoi(v) : d; }
static int kh_mpi_seq = 0;
static inline int MPI_Initialized(int *flag) { *flag = 1; return MPI_SUCCESS; }
static inline int MPI_Init(int *argc, char ***argv) { (void)argc; (void)argv; return MPI_SUCCESS; }
static inline int MPI_Comm_rank(MPI_Comm c, int *rank) { (void)c; *rank = kh_mpi_env("RANK", 0); return MPI_SUCCESS; }
static inline int MPI_Comm_size(MPI_Comm c, int *size) { (void)c; *size = kh_mpi_env("WORLD_SIZE", 1); return MPI_SUCCESS; }
static inline int MPI_Finalize(void) { return MPI_SUCCESS; }
static inline int MPI_Bcast(void *buf, int count, MPI_Datatype t, int root, MPI_Comm c) {
  (void)t; (void)c;
  int rank = kh_mpi_env("RANK", 0), size = kh_mpi_env("WORLD_SIZE", 1);
  if (size <= 1) return MPI_SUCCESS;
  char path[256], tmp[300];
  const char *job = getenv("TORCHELASTIC_RUN_ID");
  snprintf(path, sizeof(path), "/tmp/kh_mpi_bcast_%s_%d_%d", job ? job : "job", kh_mpi_env("MASTER_PORT", 0), kh_mpi_seq++);
  if (rank == root) {
    snprintf(tmp, sizeof(tmp), "%s.tmp", path);
    FILE *f = fopen(tmp, "wb");
    if (!f || fwrite(buf, 1, (size_t)count, f) != (size_t)count) { fprintf(stderr, "mpi shim: cannot write %s\n", tmp); exit(1); }
    fclose(f);
    rename(tmp, path);
  } else {
    for (int tries = 0; tries < 60000; tries++) {      /* up to 60 s */
      FILE *f = fopen(path, "rb");
      if (f) {
        size_t n = fread(buf, 1, (size_t)count, f);
        fclose(f);
        if (n == (size_t)count) return MPI_SUCCESS;
      }
      usleep(1000);
    }
    fprintf(stderr, "mpi shim: rank %d timed out waiting for %s\n", rank, path);
    exit(1);
  }
  return MPI_SUCCESS;
}
#endif
