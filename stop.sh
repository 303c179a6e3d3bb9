#!/usr/bin/env bash
# Stop the server that ./run.sh started: SIGTERM to the recorded process group, SIGKILL after a grace period.
#   ./stop.sh [--grace SECONDS]
set -euo pipefail
root="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
grace=20
[ "${1:-}" = "--grace" ] && grace="$2"
pidfile="$root/ds41rt.pid"
[ -f "$pidfile" ] || { echo "not running (no $pidfile)"; exit 0; }
pgid="$(cat "$pidfile")"
case "$pgid" in ''|*[!0-9]*) echo "bad pid file" >&2; exit 1 ;; esac
if kill -0 "-$pgid" 2>/dev/null; then
  kill -TERM "-$pgid"
  for _ in $(seq "$grace"); do
    kill -0 "-$pgid" 2>/dev/null || break
    sleep 1
  done
  kill -0 "-$pgid" 2>/dev/null && kill -KILL "-$pgid"
  echo "stopped process group $pgid"
else
  echo "process group $pgid is not running"
fi
rm -f "$pidfile"
