#!/bin/sh
# Install the unmodified reference (nilesh2797/BlockRank) into baseline/_ref with pip, offline.
#   sh baseline/install_ref.sh /path/to/BlockRank-checkout
# The checkout may be read-only (setuptools writes build files next to setup.py), so it is copied
# to a scratch directory first.  --no-deps: the reference's requirements (trl, peft, pytrec_eval,
# deepspeed, ...) are training-only and absent from this image; the prefill path needs torch,
# transformers and triton, which are installed.  baseline/_ref is not tracked by git.
set -e
SRC="${1:?usage: sh baseline/install_ref.sh /path/to/BlockRank-checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
cp -r "$SRC" "$TMP/ref"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" --upgrade "$TMP/ref"
rm -rf "$TMP"
ls "$HERE/_ref/blockrank"
