#!/bin/bash
# moonlight-16b-grpo: run from the repository root.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=moonlight-16b-grpo
launch grpo --config-file template/grpo_megatron.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    models.policy_trainer.num_gpu=${num_device} \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Moonlight-16B-A3B/ \
    models.policy_trainer.context_parallel_size=2 \
    models.policy_trainer.tensor_model_parallel_size=2 \
    models.policy_trainer.expert_tensor_parallel_size=2 \
    models.policy_trainer.expert_model_parallel_size=2 \
    models.policy.max_response_tokens_length=8192 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
