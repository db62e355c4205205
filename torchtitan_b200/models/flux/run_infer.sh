#!/usr/bin/bash
# Generate images for a prompt file from a trained FLUX checkpoint, one process per GPU: the training launcher with the
# inference entry point as its program.
#   NGPU=4 CONFIG=flux_dev ./torchtitan_b200/models/flux/run_infer.sh --inference.prompts_path my_prompts.txt
here=$(dirname "$(readlink -f "$0")")
TRAIN_FILE=torchtitan_b200.models.flux.inference.infer MODULE=${MODULE:-flux} CONFIG=${CONFIG:-flux_debugmodel} \
    exec "$here/../../../run_train.sh" --checkpoint.enable --checkpoint.exclude_from_loading=lr_scheduler,dataloader,optimizer "$@"
