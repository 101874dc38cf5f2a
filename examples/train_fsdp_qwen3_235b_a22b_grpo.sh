#!/bin/bash
# qwen3-235b-a22b-fsdp-grpo: run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-235b-a22b-fsdp-grpo
launch grpo --config-file template/grpo_fsdp.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    runtime_args.sample_per_episode=2048 \
    runtime_args.train_global_batch_size=2048 \
    models.policy_trainer.num_gpu=$((num_device * ${NNODES:-8})) \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-235B-A22B/ \
    models.policy_trainer.reshard_after_forward=True \
    models.policy_trainer.gradient_checkpointing=True \
    models.policy.tensor_model_parallel_size=1 \
    models.policy.expert_model_parallel_size=8 \
    models.policy.max_response_tokens_length=2048 \
    models.policy.num_inference_per_prompt=32 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
