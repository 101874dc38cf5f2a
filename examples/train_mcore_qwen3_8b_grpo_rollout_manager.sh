#!/bin/bash
# qwen3-8b-mcore-grpo-rm: run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-8b-mcore-grpo-rm
launch grpo --config-file template/grpo_megatron.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-8B/ \
    models.policy_trainer.tensor_model_parallel_size=2 \
    runtime_args.use_rollout_manager=True \
    runtime_args.data_rerank=False \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
