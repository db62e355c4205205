#!/usr/bin/bash
# Generate images for a prompt file from a trained FLUX checkpoint, one process per GPU.
#   NGPU=4 CONFIG=flux_dev ./torchtitan_b200/models/flux/run_infer.sh --inference.prompts_path my_prompts.txt
set -ex
NGPU=${NGPU:-"8"}
export LOG_RANK=${LOG_RANK:-0}
MODULE=${MODULE:-"flux"}
CONFIG=${CONFIG:-"flux_debugmodel"}

PYTORCH_ALLOC_CONF="expandable_segments:True" \
python3 -m torch.distributed.run --nproc_per_node="${NGPU}" --rdzv_backend c10d --rdzv_endpoint="127.0.0.1:0" \
    --local-ranks-filter "${LOG_RANK}" --role rank --tee 3 \
    -m torchtitan_b200.models.flux.inference.infer --module "${MODULE}" --config "${CONFIG}" \
    --checkpoint.enable --checkpoint.exclude_from_loading=lr_scheduler,dataloader,optimizer "$@"
