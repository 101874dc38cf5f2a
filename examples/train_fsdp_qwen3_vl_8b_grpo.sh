#!/bin/bash
# qwen3-vl-8b-grpo: vision-language model (dense 8B language model, deep-stack vision features); run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-vl-8b-grpo
launch grpo --config-file template/grpo_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.model_type=vlm \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/geo3k/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/geo3k/test.json \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-VL-8B-Instruct/ \
    models.policy.max_response_tokens_length=2048 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
