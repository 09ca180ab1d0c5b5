#!/bin/bash
# Build the sm_100a kernel library in-tree and a wheel of the package (the counterpart of the reference's build.sh).
#   bash build.sh            kernels + wheel under dist/
#   bash build.sh kernels    kernels only
set -e
cd "$(dirname "$0")"
python -m mindformers_b200.ops.build
if [ "$1" != "kernels" ]; then
  python -m pip wheel --no-deps --no-build-isolation -w dist . 
fi
