#!/bin/bash
# qwen2.5-vl-7b-grpo-agent: agent task (geometry problems with an answer-checking tool) on a vision-language
# model through the rollout manager; run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen2.5-vl-7b-grpo-agent
launch grpo --config-file template/grpo_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.model_type=vlm \
    runtime_args.task_type=agent \
    runtime_args.use_rollout_manager=True \
    runtime_args.raw_chat=True \
    runtime_args.data_rerank=False \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/geo3k/train_agent.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/geo3k/test_agent.json \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen2.5-VL-7B-Instruct/ \
    models.policy.max_response_tokens_length=2048 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
