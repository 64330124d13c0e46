#!/bin/bash
# Install the unmodified reference (anminliu/VecAttention) into baseline/_ref, offline.
#
#   baseline/install_reference.sh /path/to/VecAttention        (or VECATTENTION_REFERENCE=/path/to/VecAttention)
#
# pip builds a wheel from a scratch copy (the checkout may be read-only) and unpacks it into
# baseline/_ref, which is git-ignored.  No dependency is resolved (--no-deps): the image supplies
# torch, triton and flashinfer.  --ignore-requires-python: the project pins Python 3.10.0 exactly.
# The project does not declare its two pickled Triton launch-config tables as package data, so the
# wheel lacks them; they are copied beside the installed kernels, where the code looks for them
# (spattn/src/kernels/vecattention_kernels.py:21).
set -euo pipefail
SRC=${1:-${VECATTENTION_REFERENCE:-}}
if [ -z "$SRC" ] || [ ! -d "$SRC/spattn" ]; then echo "usage: $0 /path/to/VecAttention" >&2; exit 2; fi
HERE=$(cd "$(dirname "$0")" && pwd)
TMP=$(mktemp -d)
cp -r "$SRC"/. "$TMP"/
python -m pip install --no-index --no-build-isolation --no-deps --ignore-requires-python --upgrade \
  --find-links /opt/wheelhouse --target "$HERE/_ref" "$TMP"
mkdir -p "$HERE/_ref/spattn/src/kernels/cache"
cp "$SRC"/spattn/src/kernels/cache/*.pkl "$HERE/_ref/spattn/src/kernels/cache/"
rm -rf "$TMP"
echo "installed into $HERE/_ref"
