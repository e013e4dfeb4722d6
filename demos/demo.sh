#!/bin/bash
# Run a demo config from the repository root:  demos/demo.sh demo-lstm.12ax [++key value ...]
set -e
cd "$(dirname "$0")/.."
name="${1:-demo-lstm.12ax}"
shift || true
exec python rnn.py "demos/${name%.config}.config" "$@"
