#!/usr/bin/bash
# Generate from a Llama checkpoint. Usage:
#   NGPU=1 CONFIG=llama3_debugmodel CHECKPOINT_DIR=./outputs/checkpoint/step-10 PROMPT="Hello" ./run_llama_generate.sh [extra args]
set -e
NGPU=${NGPU:-"1"}
MODULE=${MODULE:-"llama3"}
CONFIG=${CONFIG:-"llama3_debugmodel"}
CHECKPOINT_DIR=${CHECKPOINT_DIR:-""}
PROMPT=${PROMPT:-""}
python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node="${NGPU}" \
    -m torchtitan_b200.scripts.generate.test_generate --module "${MODULE}" --config "${CONFIG}" \
    --checkpoint "${CHECKPOINT_DIR}" --prompt "${PROMPT}" "$@"
