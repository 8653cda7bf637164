#!/bin/sh
# Puts the unmodified reference package where the same-box baseline (ref_triton_b200.py) imports it from:
# baseline/_ref/ (ignored by git, so the history stays free of reference sources).  The reference tree has no
# pyproject/setup.py, so `pip install --target` has nothing to build; its pure-Python package directory is taken as is.
set -e
here=$(cd "$(dirname "$0")" && pwd)
src=${1:?usage: install_ref.sh <path of the reference checkout>}
rm -rf "$here/_ref"
mkdir -p "$here/_ref"
if ! python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse --target "$here/_ref" "$src" >"$here/_ref/pip.log" 2>&1; then
    echo "pip install failed (see baseline/_ref/pip.log): copying the package directory" >&2
    cp -r "$src/ixrun" "$here/_ref/ixrun"
fi
find "$here/_ref" -name __pycache__ -type d -prune -exec rm -rf {} +
ls "$here/_ref"
