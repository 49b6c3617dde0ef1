#!/bin/bash
# Builds the unmodified reference sources for sm_100 under baseline/_ref (git-ignored):
# `make ARCH=sm_100 all tp`, with g++ plus the header-only MPI stand-in in place of mpicxx.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
SRC="${1:-/root/reference}"
DST="$HERE/_ref"
mkdir -p "$DST"
cp -r "$SRC/src" "$SRC/bench" "$SRC/tests" "$SRC/Makefile" "$DST/"
cat > "$DST/mpicxx" <<EOS
#!/bin/bash
exec g++ -I"$HERE/mpi_shim" "\$@"
EOS
chmod +x "$DST/mpicxx"
cd "$DST"
make -j8 ARCH=sm_100 NVCC="nvcc -I$HERE/mpi_shim" train bench 2>&1 | tail -3
make -j8 ARCH=sm_100 NVCC="nvcc -I$HERE/mpi_shim" MPICXX=g++ tp 2>&1 | tail -3
ls build/*.exe
