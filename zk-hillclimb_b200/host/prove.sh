#!/bin/bash
# prove.sh <run_dir>: proves every obligation of <run_dir>/public.json (needs a GPU), the prover entry point of the
# reference's harness (harness/score.py:126-147).
set -e
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
exec python "$here/../p3walk.py" prove "$1"
