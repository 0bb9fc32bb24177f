#!/bin/bash
# Puts the unmodified reference under baseline/_ref/ (git-ignored; it travels to a GPU box with the
# working tree) so that baseline/run_reference_kernels.py can time the reference's own GPU kernels as
# single-GPU comparators.  Usage: baseline/install_reference.sh /path/to/reference-checkout
#
# The reference's pyproject.toml packages only its (empty) `svdquant_kernels` stub; the kernels live
# in plain top-level Python packages (cute_kernels/, triton_kernels/, baseline/) that its own scripts
# import with the checkout on sys.path.  So: the prescribed pip install first (from a copy, the build
# writes into its tree), then those three package directories are copied as they are.
set -e
SRC="${1:?path to the reference checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
DST="$HERE/_ref"
rm -rf /tmp/_ref_src && cp -r "$SRC" /tmp/_ref_src
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$DST" /tmp/_ref_src || echo "pip install failed (recorded); copying the kernel packages only"
mkdir -p "$DST"
for pkg in cute_kernels triton_kernels baseline; do
  rm -rf "$DST/$pkg"
  cp -r "$SRC/$pkg" "$DST/$pkg"
done
find "$DST" -name "__pycache__" -type d -prune -exec rm -rf {} +
echo "reference installed under $DST"
