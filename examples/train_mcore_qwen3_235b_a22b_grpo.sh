#!/bin/bash
# qwen3-235b-a22b-grpo: multi-node (NNODES x 8 GPUs, at least 4 nodes); run on every node from the repository
# root with NODE_RANK / NNODES / MASTER_ADDR / MASTER_PORT set by the job environment.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=qwen3-235b-a22b-grpo
launch grpo --config-file template/grpo_megatron.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    runtime_args.sample_per_episode=2048 \
    runtime_args.train_global_batch_size=2048 \
    models.policy_trainer.num_gpu=$((num_device * ${NNODES:-4})) \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/Qwen3-235B-A22B/ \
    models.policy_trainer.tensor_model_parallel_size=4 \
    models.policy_trainer.pipeline_model_parallel_size=4 \
    models.policy_trainer.expert_tensor_parallel_size=1 \
    models.policy_trainer.expert_model_parallel_size=8 \
    models.policy.tensor_model_parallel_size=1 \
    models.policy.expert_model_parallel_size=8 \
    models.policy.max_response_tokens_length=2048 \
    models.policy.num_inference_per_prompt=32 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
