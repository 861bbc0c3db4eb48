#!/bin/bash
# Line and branch coverage of the device-free suite (needs the `coverage` package; prints how to proceed without it).
# Usage: bash tests/run_coverage.sh [extra pytest arguments]
cd "$(dirname "$0")/.." || exit 1
if ! python -c "import coverage" 2>/dev/null; then
  echo "the 'coverage' package is not installed; running the suite without it"
  exec python -m pytest tests/ -q -m "not gpu" "$@"
fi
python -m coverage run --branch --source=mindspeed_rl_b200 -m pytest tests/ -q -m "not gpu" "$@"
status=$?
python -m coverage report --skip-empty | tail -40
python -m coverage html -d coverage_html >/dev/null 2>&1
exit $status
