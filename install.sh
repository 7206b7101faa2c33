#!/usr/bin/env bash
# Editable install plus the in-tree build of the native libraries (nvcc for sm_100a,
# g++); the libraries stay under hipress_b200/_native/, next to the sources that
# load them.  The reference's counterpart is `bash ./install.sh` of its CaSync tree.
set -euo pipefail
cd "$(dirname "$0")"
python -m pip install --no-build-isolation --no-deps -e .
python -m hipress_b200._native.build
