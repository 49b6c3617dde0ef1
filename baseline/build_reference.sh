#!/bin/bash
# Builds the unmodified reference sources for sm_100 under baseline/_ref (git-ignored):
# `make ARCH=sm_100 all tp`, with g++ plus the header-only MPI stand-in in place of mpicxx.
#   usage: baseline/build_reference.sh <reference checkout>      (or KHARON_REFERENCE_SRC=<path>)
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
SRC="${1:-$KHARON_REFERENCE_SRC}"
if [ -z "$SRC" ] || [ ! -f "$SRC/Makefile" ]; then
  echo "usage: $0 <path of the reference checkout> (or set KHARON_REFERENCE_SRC)" >&2
  exit 2
fi
DST="$HERE/_ref"
mkdir -p "$DST"
cp -r "$SRC/src" "$SRC/bench" "$SRC/tests" "$SRC/Makefile" "$DST/"
cat > "$DST/mpicxx" <<EOS
#!/bin/bash
exec g++ -I"$HERE/mpi_shim" "\$@"
EOS
chmod +x "$DST/mpicxx"
cd "$DST"
make -j8 ARCH=sm_100 NVCC="nvcc -I$HERE/mpi_shim" train bench tests 2>&1 | tail -3
make -j8 ARCH=sm_100 NVCC="nvcc -I$HERE/mpi_shim" MPICXX=g++ tp 2>&1 | tail -3
ls build/*.exe
