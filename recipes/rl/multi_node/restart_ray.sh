#!/usr/bin/env bash
# Brings this run's Ray cluster up (again) on the nodes of a multi-node job: on every node it stops the Ray processes
# that belong to the run's private temp dir (and only those -- other users' clusters on shared machines are not
# touched), starts the head on the first host and a worker on each remaining host, and waits until all GPUs are
# registered.
#   HOSTS="node0 node1 node2 node3" GPUS_PER_NODE=8 ARL_RAY_TEMP_DIR=/tmp/arl-ray-myrun ./restart_ray.sh
# Start commands (port, temp dir, worker port range from ARL_RAY_MIN_WORKER_PORT / ARL_RAY_MAX_WORKER_PORT) come from
# `python -m arctic_platform_b200.common.ray_cluster`; the other nodes are reached with ssh.
set -euo pipefail
HOSTS=(${HOSTS:?space-separated host names, head first})
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
PORT=${RAY_PORT:-6379}
TMP=${ARL_RAY_TEMP_DIR:?a temp dir private to this run (it identifies the cluster)}
HEAD=${HOSTS[0]}
RC="python -m arctic_platform_b200.common.ray_cluster"

for h in "${HOSTS[@]}"; do ssh "$h" "$RC stop --temp-dir $TMP" || true; done
ssh "$HEAD" "\$($RC head --port $PORT --temp-dir $TMP --num-gpus $GPUS_PER_NODE)"
for h in "${HOSTS[@]:1}"; do
  ssh "$h" "\$($RC worker --head-address $HEAD:$PORT --temp-dir $TMP --num-gpus $GPUS_PER_NODE)"
done

want=$(( ${#HOSTS[@]} * GPUS_PER_NODE ))
have=0
for _ in $(seq 1 60); do
  have=$(ssh "$HEAD" "python -c \"import ray; ray.init(address='$HEAD:$PORT', logging_level='ERROR'); print(int(ray.cluster_resources().get('GPU', 0)))\"" 2>/dev/null || echo 0)
  if [ "$have" -ge "$want" ]; then echo "ray cluster ready: $have GPUs on ${#HOSTS[@]} nodes"; exit 0; fi
  sleep 5
done
echo "ray cluster incomplete: $have of $want GPUs" >&2
exit 1
