#!/bin/bash
# Gather the per-rank expert-load dumps of a multi-node run on this node.  Every rollout rank writes
# its token counts per expert as JSON under generate_config.eplb_token_save_path
# (generate_config.eplb_token_collects: true); copy them from the
# other nodes before generating the placement map.
# Usage: bash examples/eplb/collect_json_file.sh <dump dir> <node> [<node> ...]
set -euo pipefail
DUMP_DIR=${1:?dump directory}
shift
for node in "$@"; do
  scp "$node:$DUMP_DIR/*.json" "$DUMP_DIR/"
done
ls "$DUMP_DIR"/*.json | wc -l
