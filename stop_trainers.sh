#!/bin/bash
# Stop the trainers started by gtopk_run.sh / dense_run.sh on this machine.
# The launchers run under torchrun, which records nothing by itself, so this
# script takes the launcher's process id (or a file holding it) and signals that
# process group only -- it never matches processes by name.
#   ./stop_trainers.sh <launcher pid | pid file>
set -e
arg="${1:?usage: stop_trainers.sh <launcher pid | pid file>}"
if [ -f "$arg" ]; then pid="$(cat "$arg")"; else pid="$arg"; fi
pgid="$(ps -o pgid= -p "$pid" | tr -d ' ')"
[ -n "$pgid" ] || { echo "no such process: $pid"; exit 1; }
kill -TERM -- "-$pgid"
echo "sent SIGTERM to process group $pgid"
