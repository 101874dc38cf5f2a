"""GRPO / GSPO algorithm: configuration, dataflow and the launcher glue.

Parity: chatlearn/algorithm/grpo.py:93-354.  The three flow functions are written
exactly as in the reference (:215-237); what differs is what executes them (the
SPMD executor) and the roles behind the names (the native rollout engine, the
FSDP-style or TP/EP-style trainers of this framework).
"""
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Any, Optional

from chatlearn_b200.algorithm.base_algo import BaseAlgorithm
from chatlearn_b200.algorithm.grpo_utils.advantage_compute import AdvantageComputer
from chatlearn_b200.configs import (BaseConfig, FSDPPolicyTrainerConfig, FSDPRefPolicyConfig,
                                    MegatronPolicyTrainerConfig, MegatronRefPolicyConfig,
                                    PartialRolloutManagerConfig, PolicyConfig, RewardConfig,
                                    RolloutManagerConfig, RuntimeConfig, RuntimeEnvConfig, to_dataclass)
from chatlearn_b200.runtime.engine import Engine
from chatlearn_b200.runtime.environment import Environment
from chatlearn_b200.runtime.evaluator import Evaluator
from chatlearn_b200.runtime.trainer import Trainer


@dataclass
class GrpoModelConfig(BaseConfig):
    policy: PolicyConfig = field(default_factory=PolicyConfig)
    reward: RewardConfig = field(default_factory=RewardConfig)
    ref_policy: Any = field(default_factory=FSDPRefPolicyConfig)
    policy_trainer: Any = field(default_factory=FSDPPolicyTrainerConfig)
    rollout_manager: Optional[RolloutManagerConfig] = None
    partial_rollout_manager: Optional[PartialRolloutManagerConfig] = None


@dataclass
class GrpoConfig(BaseConfig):
    env_args: RuntimeEnvConfig = field(default_factory=RuntimeEnvConfig)
    runtime_args: RuntimeConfig = field(default_factory=RuntimeConfig)
    models: GrpoModelConfig = field(default_factory=GrpoModelConfig)

    def _post_init_impl(self):
        backend = self.runtime_args.train_backend
        m = self.models
        ref_cls, tr_cls = {
            "megatron": (MegatronRefPolicyConfig, MegatronPolicyTrainerConfig),
        }.get(backend, (FSDPRefPolicyConfig, FSDPPolicyTrainerConfig))
        if isinstance(m.ref_policy, dict):
            m.ref_policy = to_dataclass(ref_cls, m.ref_policy, "models.ref_policy")
        if isinstance(m.policy_trainer, dict):
            m.policy_trainer = to_dataclass(tr_cls, m.policy_trainer, "models.policy_trainer")
        if m.policy_trainer is not None:
            m.policy_trainer.trainable = True

    def _validate_impl(self):
        ra, m = self.runtime_args, self.models
        n = int(ra.num_inference_per_prompt)
        assert ra.sample_per_episode % n == 0, \
            "sample_per_episode must be a multiple of num_inference_per_prompt"
        assert ra.sample_per_episode % ra.train_global_batch_size == 0, \
            "sample_per_episode must be a multiple of train_global_batch_size"
        pol = m.policy
        dp_rollout = max(pol.num_replica, 1) * max(pol.expert_model_parallel_size, 1)
        assert ra.sample_per_episode % dp_rollout == 0, \
            "sample_per_episode must divide evenly over the rollout replicas"
        tr = m.policy_trainer
        dp_train = int(tr.replica_dp_size or 1) * max(int(tr.num_replica or 1), 1)
        assert ra.train_global_batch_size % dp_train == 0, \
            f"train_global_batch_size must be a multiple of the trainer data-parallel size {dp_train}"
        if not tr.packing:
            assert (ra.train_global_batch_size // dp_train) % ra.train_micro_batch_size == 0, \
                "per-rank batch must be a multiple of train_micro_batch_size"
        if ra.use_partial_rollout:
            assert m.partial_rollout_manager is not None, "use_partial_rollout needs models.partial_rollout_manager"
        if ra.use_rollout_manager:
            assert m.rollout_manager is not None, "use_rollout_manager needs models.rollout_manager"


class GRPOEvaluator(Evaluator):
    def post_process(self, results, eval_info):
        stats = defaultdict(list)
        max_resp = self.global_args.models.policy.max_response_tokens_length
        for batch in results.get("reward", []):
            for r in batch:
                key = r.get("eval_source", "")
                stats[f"eval_{key}"].append(r["rule_reward"])
                stats[f"eval_{key}_response_length"].append(r["response_token_length"])
                stats[f"eval_{key}_response_clip_ratio"].append(float(r["response_token_length"] >= max_resp))
        self._metric_list.append({k: sum(v) / len(v) for k, v in stats.items() if v})
        return results


class GRPOEngine(Engine):
    def __init__(self, policy, reward, ref_policy, policy_trainer, partial_rollout_manager=None):
        def env_compute_flow(batch):
            policy_out = policy.forward_step(batch)
            old_logprobs_out = policy_trainer.forward_step(policy_out)
            ref_logprobs_out = ref_policy.forward_step(old_logprobs_out)
            reward_out = reward.forward_step(ref_logprobs_out)
            return reward_out

        def env_compute_flow_partial(batch):
            batch = partial_rollout_manager.get_sample_for_rollout(batch)
            batch = policy.forward_step(batch)
            batch = partial_rollout_manager.post_process_rollout_results(batch)
            old_logprobs_out = policy_trainer.forward_step(batch)
            ref_logprobs_out = ref_policy.forward_step(old_logprobs_out)
            reward_out = reward.forward_step(ref_logprobs_out)
            return reward_out

        def trainer_compute_flow(batch):
            policy_trainer.train_step(batch)

        def evaluator_flow(batch):
            policy_out = policy.eval_forward(batch)
            reward_out = reward.eval_forward(policy_out)
            return reward_out

        models = [policy, reward, ref_policy, policy_trainer]
        if partial_rollout_manager is not None:
            env = Environment(env_compute_flow_partial)
            models.append(partial_rollout_manager)
        else:
            env = Environment(env_compute_flow)
        super().__init__(environment=env, trainer=Trainer(trainer_compute_flow),
                         evaluator=GRPOEvaluator(evaluator_flow), name="grpo", models=models)
        self.set_parameter_sync(policy_trainer, policy)


class RolloutManagerGRPOEngine(Engine):
    def __init__(self, rollout_manager, policy, reward, ref_policy, policy_trainer):
        def env_compute_flow(batch):
            rollout_out = rollout_manager.forward_step(batch)
            old_logprobs_out = policy_trainer.forward_step(rollout_out)
            ref_logprobs_out = ref_policy.forward_step(old_logprobs_out)
            reward_out = reward.forward_step(ref_logprobs_out)
            return reward_out

        def trainer_compute_flow(batch):
            policy_trainer.train_step(batch)

        def evaluator_flow(batch):
            rollout_out = rollout_manager.eval_forward(batch)
            reward_out = reward.eval_forward(rollout_out)
            return reward_out

        super().__init__(environment=Environment(env_compute_flow), trainer=Trainer(trainer_compute_flow),
                         evaluator=GRPOEvaluator(evaluator_flow), name="grpo",
                         models=[rollout_manager, policy, reward, ref_policy, policy_trainer])
        self.set_parameter_sync(policy_trainer, policy)


class GrpoAlgorithm(BaseAlgorithm):
    def __init__(self, cfg: GrpoConfig):
        if cfg.runtime_args.train_backend == "megatron":
            from chatlearn_b200.utils.megatron_utils import update_cfg
            cfg = update_cfg(cfg)
        self.cfg = cfg
        self.engine = None

    def validate(self):
        self.cfg.validate()

    def build_engine(self):
        import chatlearn_b200
        from chatlearn_b200.data.data import read_data_path_list
        from chatlearn_b200.models.reward.rule_reward import RuleReward
        from chatlearn_b200.models.rollout_module import RolloutModule
        cfg = self.cfg
        chatlearn_b200.init(cfg)
        ra = cfg.runtime_args
        if ra.train_backend == "fsdp":
            from chatlearn_b200.algorithm.grpo_utils.policy_trainer import PolicyTrainer as T
        else:
            from chatlearn_b200.algorithm.grpo_utils.megatron_policy_trainer import MegatronPolicyTrainer as T
        policy_trainer, ref_policy = T("policy_trainer"), T("ref_policy")
        if ra.task_type == "agent":
            from chatlearn_b200.models.agent.agent_module import AgentModule
            assert ra.use_rollout_manager, "agent tasks run through the rollout manager"
            policy = AgentModule("policy")
        else:
            policy = RolloutModule("policy")
        reward = RuleReward("reward")
        if ra.use_rollout_manager:
            from chatlearn_b200.models.agent.rollout_manager import RolloutManager
            engine = RolloutManagerGRPOEngine(RolloutManager("rollout_manager", engine_module=policy), policy, reward,
                                              ref_policy, policy_trainer)
        else:
            prm = None
            if ra.use_partial_rollout:
                from chatlearn_b200.algorithm.grpo_utils.partial_rollout_manager import PartialRolloutManager
                prm = PartialRolloutManager("partial_rollout_manager")
            engine = GRPOEngine(policy, reward, ref_policy, policy_trainer, prm)
        train = read_data_path_list([p.strip() for p in ra.data_path.split(",")])
        engine.set_dataset(train)
        if ra.eval_data_path:
            engine.evaluator.set_dataset(
                read_data_path_list([p.strip() for p in ra.eval_data_path.split(",")]))
        else:
            engine.evaluator = None
        engine.set_replay_sample_manager(AdvantageComputer(ra.num_inference_per_prompt))
        self.engine = engine
        return engine

    def run(self):
        return self.build_engine().learn()
