#!/usr/bin/env bash
# Pin a rank to the NUMA node of its GPU when numactl is available (reference: numa_wrapper.sh:16-17).
if command -v numactl >/dev/null 2>&1 && [ -n "${LOCAL_RANK:-}" ]; then
    NODES=$(numactl --hardware | awk '/available:/ {print $2}')
    NODE=$(( LOCAL_RANK * NODES / ${LOCAL_WORLD_SIZE:-8} ))
    exec numactl --cpunodebind="$NODE" --membind="$NODE" "$@"
fi
exec "$@"
