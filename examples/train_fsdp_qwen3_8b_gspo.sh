#!/bin/bash
# qwen3-8b-gspo: run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-8b-gspo
launch grpo --config-file template/grpo_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-8B/ \
    models.policy_trainer.use_group_sequence_policy=True \
    models.policy_trainer.pos_clip_ratio=4e-4 \
    models.policy_trainer.neg_clip_ratio=3e-4 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
