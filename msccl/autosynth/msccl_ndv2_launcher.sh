#!/bin/bash
# Launch a command on an NDv2 with GPUs re-ordered to the canonical DGX-1 numbering.
# msccl.ndv2_perm() caches the order in the lock file read below.
lock=/var/lock/msccl_autosynth_inspector_topo.lock
python -c "import msccl; msccl.ndv2_perm()"
if [ -f "$lock" ]; then
    CUDA_VISIBLE_DEVICES=$(cat "$lock")
    export CUDA_VISIBLE_DEVICES
    echo "Set CUDA_VISIBLE_DEVICES to: $CUDA_VISIBLE_DEVICES"
fi
exec "$@"
