#!/bin/bash
# verify.sh <proof_dir> <public.json> <transcript-out>: the verifier entry point of the reference's harness
# (harness/score.py:149-186): exit 0 = ACCEPT; the transcript lists the manifest ids that were checked.
set -e
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
exec python "$here/../p3walk.py" verify "$1" "$2" "$3"
