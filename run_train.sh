#!/usr/bin/bash
# Launch a training job on one node, one process per GPU.
#   NGPU=8 MODULE=llama3 CONFIG=llama3_8b ./run_train.sh --training.steps 100
# COMM_MODE=fake_backend validates configuration, meshes and parallelisation without GPUs;
# COMM_MODE=local_tensor runs a single process for debugging.
set -ex
NGPU=${NGPU:-"8"}
export LOG_RANK=${LOG_RANK:-0}
MODULE=${MODULE:-"llama3"}
CONFIG=${CONFIG:-"llama3_debugmodel"}
TRAIN_FILE=${TRAIN_FILE:-"torchtitan_b200.train"}
COMM_MODE=${COMM_MODE:-""}

if [ -n "$COMM_MODE" ]; then
    echo "Running with comm_mode=${COMM_MODE}"
    NGPU="${NGPU}" LOCAL_RANK=0 python3 -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" \
        "$@" --comm.mode="${COMM_MODE}" --training.steps=1
else
    PYTORCH_ALLOC_CONF="expandable_segments:True" \
    python3 -m torch.distributed.run --nproc_per_node="${NGPU}" --rdzv_backend c10d --rdzv_endpoint="127.0.0.1:0" \
        --local-ranks-filter "${LOG_RANK}" --role rank --tee 3 \
        -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" "$@"
fi
