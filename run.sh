#!/usr/bin/env bash
# Start the server on this node: one process per GPU, rank 0 serves HTTP, the others mirror its engine calls.
#
#   ./run.sh [--gpus N] [--select "OPTIONS"] [--settings FILE] [--log FILE] [--foreground] [-- any `serve` option ...]
#
# --select picks the N GPUs with the most free memory that can hold the launch and exports them as
# CUDA_VISIBLE_DEVICES; OPTIONS go to `python -m ds41rt_b200 select-gpus` (e.g. "--model flash --concurrency 16
# --max-context 32768 --reclaim-pid 4242"; "" for its defaults).  Without it the first N visible GPUs are used.
# Options after `--` go to `python -m ds41rt_b200 serve` unchanged and override the settings file and the DS41RT_<KEY>
# environment (the three tiers of ds41rt_b200/settings.py).  The launch is recorded in ./ds41rt.pid (process-group id
# of the launcher), which ./stop.sh reads; the rendezvous stays on 127.0.0.1.
set -euo pipefail
root="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
gpus=1; settings=""; log="$root/ds41rt.log"; foreground=0; select=0; select_opts=""
while [ $# -gt 0 ]; do
  case "$1" in
    --gpus) gpus="$2"; shift 2 ;;
    --select) select=1; select_opts="$2"; shift 2 ;;
    --settings) settings="$2"; shift 2 ;;
    --log) log="$2"; shift 2 ;;
    --foreground) foreground=1; shift ;;
    -h|--help) sed -n '2,11p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; exit 0 ;;
    --) shift; break ;;
    *) echo "unknown option: $1 (serve options go after --)" >&2; exit 64 ;;
  esac
done
case "$gpus" in 1|2|4|8) ;; *) echo "--gpus must be 1, 2, 4 or 8" >&2; exit 64 ;; esac
if [ -f "$root/ds41rt.pid" ] && kill -0 "-$(cat "$root/ds41rt.pid")" 2>/dev/null; then
  echo "already running (process group $(cat "$root/ds41rt.pid")); ./stop.sh first" >&2; exit 1
fi
cd "$root"
python -m ds41rt_b200 build >/dev/null
if [ "$select" -eq 1 ]; then
  # shellcheck disable=SC2086  # the option string is split into words on purpose
  CUDA_VISIBLE_DEVICES="$(python -m ds41rt_b200 select-gpus --gpus "$gpus" --print-devices $select_opts)"
  export CUDA_VISIBLE_DEVICES
  echo "GPUs: $CUDA_VISIBLE_DEVICES"
fi
args=(serve)
[ -n "$settings" ] && args+=(--settings "$settings")
args+=("$@")
if [ "$gpus" -eq 1 ]; then
  cmd=(python -m ds41rt_b200 "${args[@]}")
else
  port=$((20000 + RANDOM % 10000))
  cmd=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$gpus" --master-addr 127.0.0.1
       --master-port "$port" -m ds41rt_b200 "${args[@]}")
fi
if [ "$foreground" -eq 1 ]; then
  exec "${cmd[@]}"
fi
setsid "${cmd[@]}" >"$log" 2>&1 &
echo $! > "$root/ds41rt.pid"          # setsid: the launcher leads its own process group, pid == pgid
echo "started process group $(cat "$root/ds41rt.pid"); log: $log"
