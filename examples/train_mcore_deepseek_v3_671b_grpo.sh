#!/bin/bash
# deepseek-v3-671b-grpo: multi-node (NNODES x 8 GPUs, at least 16 nodes); run on every node from the repository
# root with NODE_RANK / NNODES / MASTER_ADDR / MASTER_PORT set by the job environment.
# Trainer: TP=4 (experts sliced over the same 4 ranks), PP=16 with 3 + 2 layers on the first / last stage, EP=2.
# Rollout: every rank keeps the attention weights and 1/32 of the experts; the cache holds one compressed
# latent row per token and decode attends in the latent space.
set -x
export CHATLEARN=$(pwd)
export PYTHONPATH=${CHATLEARN}:${PYTHONPATH}
source examples/base_env.sh
export exp_name=deepseek-v3-671b-grpo
launch grpo --config-file template/grpo_megatron.yaml \
    runtime_args.exp_name=${exp_name} \
    runtime_args.output_dir=${CHATLEARN}/output/${exp_name} \
    runtime_args.data_path=${CHATLEARN}/dataset/MATH-lighteval/train.json \
    runtime_args.eval_data_path=${CHATLEARN}/dataset/MATH-lighteval/test.json \
    runtime_args.sample_per_episode=256 \
    runtime_args.train_global_batch_size=256 \
    models.policy_trainer.num_gpu=$((num_device * ${NNODES:-16})) \
    models.policy_trainer.load=${CHATLEARN}/pretrained_models/DeepSeek-V3/ \
    models.policy_trainer.tensor_model_parallel_size=4 \
    models.policy_trainer.pipeline_model_parallel_size=16 \
    models.policy_trainer.decoder_first_pipeline_num_layers=3 \
    models.policy_trainer.decoder_last_pipeline_num_layers=2 \
    models.policy_trainer.expert_tensor_parallel_size=4 \
    models.policy_trainer.expert_model_parallel_size=2 \
    models.policy_trainer.context_parallel_size=1 \
    models.policy.expert_model_parallel_size=32 \
    models.policy.max_response_tokens_length=2048 \
    models.policy.num_inference_per_prompt=32 \
    2>&1 | tee ${CHATLEARN}/output_${exp_name}.log
