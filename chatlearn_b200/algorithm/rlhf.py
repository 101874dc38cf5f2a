"""PPO-style RLHF with a learned reward model (and optionally a critic).

Parity: the six-role dataflow of ``RLHFEngine`` (chatlearn/runtime/engine.py:601-626:
policy, reference, reward, value inference; policy and value trainers) and the
README's "N+N" policy + reward set-up.  Two shapes are supported:

* **three models** (``models.value_trainer`` absent): policy rollout → behaviour
  log-probs (policy trainer) → reference log-probs → reward model score.  The
  advantage of a response is its KL-shaped return, group-normalised when a prompt
  has several samples and batch-whitened otherwise; the update is the clipped
  policy-gradient objective shared with GRPO.
* **actor–critic** (``models.value_trainer`` present): a critic with a scalar head
  gives per-token values, advantages come from GAE(γ, λ), the critic is trained on
  the clipped value loss.  The critic scores with the weights it trains, so no
  separate value-inference role or parameter sync is needed; ``RLHFEngine`` with
  six roles remains available for users who want that placement.

Per-token reward: ``r_t = -β (log π_old − log π_ref)_t``, plus the clipped
reward-model score on the last response token.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from chatlearn_b200.algorithm.base_algo import BaseAlgorithm
from chatlearn_b200.algorithm.grpo_utils.policy_trainer import PolicyTrainer
from chatlearn_b200.algorithm.grpo_utils.trainer_utils import pack_samples, unpack_per_sample
from chatlearn_b200.configs import (BaseConfig, FSDPPolicyTrainerConfig, FSDPRefPolicyConfig, PolicyConfig,
                                    RuntimeConfig, RuntimeEnvConfig, to_dataclass)
from chatlearn_b200.data.data import ReplaySampleManager
from chatlearn_b200.models.nn.model import FwdCtx
from chatlearn_b200.runtime.engine import Engine
from chatlearn_b200.runtime.environment import Environment
from chatlearn_b200.runtime.trainer import Trainer
from chatlearn_b200.utils import xfer


@dataclass
class RlhfModelConfig(BaseConfig):
    policy: PolicyConfig = field(default_factory=PolicyConfig)
    reference: Any = field(default_factory=FSDPRefPolicyConfig)
    reward: Any = field(default_factory=FSDPRefPolicyConfig)
    policy_trainer: Any = field(default_factory=FSDPPolicyTrainerConfig)
    value_trainer: Optional[Any] = None


@dataclass
class RlhfConfig(BaseConfig):
    env_args: RuntimeEnvConfig = field(default_factory=RuntimeEnvConfig)
    runtime_args: RuntimeConfig = field(default_factory=RuntimeConfig)
    models: RlhfModelConfig = field(default_factory=RlhfModelConfig)

    def _post_init_impl(self):
        m = self.models
        for name, cls in (("reference", FSDPRefPolicyConfig), ("reward", FSDPRefPolicyConfig),
                          ("policy_trainer", FSDPPolicyTrainerConfig), ("value_trainer", FSDPPolicyTrainerConfig)):
            v = getattr(m, name)
            if isinstance(v, dict):
                setattr(m, name, to_dataclass(cls, v, f"models.{name}"))
        m.policy_trainer.trainable = True
        # advantages are computed by the replay sample manager, which runs on the replay window
        if int(self.runtime_args.max_replay_episode or 0) == 0:
            self.runtime_args.max_replay_episode = 1
        if m.value_trainer is not None:
            m.value_trainer.trainable = True

    def _validate_impl(self):
        ra = self.runtime_args
        assert ra.train_backend == "fsdp", "the RLHF recipe uses the ZeRO (fsdp) trainer backend"
        assert ra.sample_per_episode % ra.train_global_batch_size == 0, \
            "sample_per_episode must be a multiple of train_global_batch_size"
        assert ra.sample_per_episode % int(ra.num_inference_per_prompt) == 0


def _score_arch(module_args):
    """The role's architecture with a scalar head instead of the LM head."""
    from chatlearn_b200.models.nn.arch import resolve_arch
    import copy
    arch = copy.copy(resolve_arch(module_args))
    arch.num_labels = 1
    return arch


class ScalarHeadModule(PolicyTrainer):
    """A causal LM with a one-output linear head on the final hidden states."""

    def create_model(self):
        from chatlearn_b200.models.nn.model import CausalLM
        ma = self.module_args
        dp = self.dp_group.size if self.dp_group is not None else 1
        model = CausalLM(_score_arch(ma), dtype=self.compute_dtype, device=self.device, pad_to=dp * 8)
        load = getattr(ma, "load", None)
        from chatlearn_b200.checkpoint.safetensors_io import has_safetensors, load_into_model
        if load and has_safetensors(load):
            load_into_model(model, load, strict=False)      # LM checkpoints have no score head
        else:
            model.init_weights(int(getattr(ma, "seed", 1234)))
        return model

    def _scores(self, batch):
        """Scalar per position of a packed row, fp32 ``[T]``."""
        batch.to(self.device)
        ctx = FwdCtx(positions=batch.positions, cu_seqlens=batch.cu_seqlens, max_seqlen=batch.max_seqlen)
        tokens = batch.tokens
        if self.sp is not None:
            ctx.sp, ctx.attn_positions = self.sp, batch.positions
            tokens = self.sp.split(tokens)
            ctx.positions = self.sp.split(batch.positions)
        hook = None
        if torch.is_grad_enabled() and getattr(self.module_args, "gradient_checkpointing", False):
            from torch.utils.checkpoint import checkpoint
            from chatlearn_b200.models.nn.model import decoder_layer
            arch = self.model.arch

            def hook(l, p, x, c):
                return checkpoint(lambda xx: decoder_layer(arch, p, xx, c, l), x, use_reentrant=False)
        h = self.model.hidden_states(tokens, ctx, hook)
        v = torch.nn.functional.linear(h, self.model.block_by_name["head"].params["score"]).float().squeeze(-1)
        return self.sp.gather(v) if self.sp is not None else v


class RewardModel(ScalarHeadModule):
    """Scores a finished response: the head's output on its last token
    (``rm_score``; clipped to ±``clip_reward_value`` when that option is set)."""

    @torch.no_grad()
    def forward_step(self, data_list: List[Dict], iteration: int = 0, **kwargs):
        if not data_list:
            return data_list
        clip = float(getattr(self.module_args, "clip_reward_value", 0.0) or 0.0)
        pad = self.sp.size if self.sp is not None else 1
        scores = []
        for mb in self._microbatches(data_list, for_train=False):
            if not mb:
                continue
            batch = pack_samples(mb, pad_multiple=pad)
            v = self._scores(batch)
            # the last real token of each sequence (any alignment pad comes after it)
            lens = torch.tensor([int(s["prompt_token_length"]) + int(s["response_token_length"]) for s in mb],
                                device=batch.cu_seqlens.device)
            last = batch.cu_seqlens[:len(mb)].long() + lens - 1
            sc = v[last.to(v.device)]
            if clip > 0:
                sc = sc.clamp(-clip, clip)
            for s, x in zip(mb, xfer.tolist(sc)):
                s["rm_score"] = float(x)
                scores.append(float(x))
        if scores:
            self._metric_list.append({"rm_score": sum(scores) / len(scores)})
        return data_list

    eval_forward = forward_step


class ValueTrainer(ScalarHeadModule):
    """Critic: ``forward_step`` adds per-response-token ``values``; ``train_step``
    minimises the clipped squared error against ``returns``."""

    @torch.no_grad()
    def forward_step(self, data_list: List[Dict], iteration: int = 0, **kwargs):
        pad = self.sp.size if self.sp is not None else 1
        for mb in self._microbatches(data_list, for_train=False):
            if not mb:
                continue
            batch = pack_samples(mb, pad_multiple=pad)
            v = self._scores(batch)
            for s, x in zip(mb, unpack_per_sample(v, batch, mb)):
                s["values"] = x
        return data_list

    def train_step(self, data_list: List[Dict], **kwargs):
        ma, st = self.module_args, self.state
        clip = float(getattr(ma, "cliprange_value", 0.2))
        n_tok = torch.tensor([float(sum(int(s["response_token_length"]) for s in data_list))], device=self.device)
        if self.role_group is not None and self.role_group.size > 1:
            self.role_group.all_reduce_(n_tok)
            if self.sp is not None:
                n_tok /= self.sp.size
        inv = 1.0 / max(float(n_tok.item()), 1.0)
        st.zero_grad()
        stats = torch.zeros(2, device=self.device)
        pad = self.sp.size if self.sp is not None else 1
        for mb in self._microbatches(data_list, for_train=True):
            if not mb:
                continue
            batch = pack_samples(mb, pad_multiple=pad)
            v = self._scores(batch)
            old, ret, m = batch.values, batch.returns, batch.loss_mask
            v_clip = old + (v - old).clamp(-clip, clip)
            loss_tok = 0.5 * torch.maximum((v - ret) ** 2, (v_clip - ret) ** 2)
            loss = (loss_tok * m).sum() * inv
            loss.backward()
            stats += torch.stack([(loss_tok.detach() * m).sum(), m.sum()])
        gn = st.step()
        if self.role_group is not None and self.role_group.size > 1:
            self.role_group.all_reduce_(stats)
        host = xfer.tolist(torch.cat([stats, gn.reshape(1).float()]))
        self._metric_list.append({"value_loss": host[0] / max(host[1], 1.0), "grad_norm": host[2]})
        self._train_iteration += 1


def gae(rewards: torch.Tensor, values: torch.Tensor, gamma: float, lam: float):
    """Generalised advantage estimation over one response (terminal value 0)."""
    n = rewards.numel()
    adv = torch.zeros(n)
    last = 0.0
    for t in range(n - 1, -1, -1):
        nxt = float(values[t + 1]) if t + 1 < n else 0.0
        delta = float(rewards[t]) + gamma * nxt - float(values[t])
        last = delta + gamma * lam * last
        adv[t] = last
    return adv, adv + values


class RlhfAdvantage(ReplaySampleManager):
    """Turns scores, log-probs (and values) of an episode into advantages (and returns)."""

    def __init__(self, kl_coef: float = 0.05, gamma: float = 1.0, lam: float = 0.95,
                 num_inference_per_prompt: int = 1, whiten: bool = True):
        super().__init__()
        self.kl_coef, self.gamma, self.lam = kl_coef, gamma, lam
        self.n, self.whiten = num_inference_per_prompt, whiten
        self._metric_prefix = "rlhf_advantage"

    def token_rewards(self, s: Dict) -> torch.Tensor:
        n = int(s["response_token_length"])
        r = torch.zeros(n)
        if self.kl_coef and "ref_logprobs" in s and "old_logprobs" in s:
            old = torch.as_tensor(s["old_logprobs"], dtype=torch.float32).flatten()[:n]
            ref = torch.as_tensor(s["ref_logprobs"], dtype=torch.float32).flatten()[:n]
            r[:old.numel()] = -self.kl_coef * (old - ref)
        if n:
            r[n - 1] += float(s["rm_score"])
        return r

    def __call__(self, episode_replay_buffers) -> List[Dict]:
        buf = episode_replay_buffers[-1].buffer
        have_values = all("values" in s for s in buf) and len(buf) > 0
        kls, rets = [], []
        for s in buf:
            r = self.token_rewards(s)
            kls.append(float(-(r.sum() - float(s["rm_score"])) / max(self.kl_coef, 1e-12)) if self.kl_coef else 0.0)
            if have_values:
                v = torch.as_tensor(s["values"], dtype=torch.float32).flatten()[:r.numel()]
                adv, ret = gae(r, v, self.gamma, self.lam)
                s["advantages"], s["returns"] = adv, ret
            else:
                s["_return"] = float(r.sum())
            rets.append(float(r.sum()))
        if have_values:
            if self.whiten:
                allv = torch.cat([s["advantages"] for s in buf])
                mean, std = allv.mean(), allv.std(unbiased=False)
                for s in buf:
                    s["advantages"] = (s["advantages"] - mean) / (std + 1e-8)
        else:
            groups: Dict[str, List[Dict]] = {}
            for s in buf:
                groups.setdefault(s["prompt_uid"] if self.n > 1 else "", []).append(s)
            for grp in groups.values():
                x = torch.tensor([g.pop("_return") for g in grp])
                mean, std = x.mean(), x.std(unbiased=False)
                for g, xi in zip(grp, x):
                    g["advantages"] = float((xi - mean) / (std + 1e-5))
        if buf:
            self._metric_list.append({"return_mean": sum(rets) / len(rets), "kl_mean": sum(kls) / len(kls)})
        return list(buf)


class ThreeModelRLHFEngine(Engine):
    """policy + reference + reward model (no critic)."""

    def __init__(self, policy, reference, reward, policy_trainer, value_trainer=None):
        def env_compute_flow(batch):
            policy_out = policy.forward_step(batch)
            old_out = policy_trainer.forward_step(policy_out)
            ref_out = reference.forward_step(old_out)
            if value_trainer is not None:
                ref_out = value_trainer.forward_step(ref_out)
            return reward.forward_step(ref_out)

        def trainer_compute_flow(batch):
            policy_trainer.train_step(batch)
            if value_trainer is not None:
                value_trainer.train_step(batch)

        models = [policy, reference, reward, policy_trainer] + ([value_trainer] if value_trainer is not None else [])
        super().__init__(environment=Environment(env_compute_flow), trainer=Trainer(trainer_compute_flow),
                         name="rlhf", models=models)
        self.set_parameter_sync(policy_trainer, policy)


class RlhfAlgorithm(BaseAlgorithm):
    def __init__(self, cfg: RlhfConfig):
        self.cfg, self.engine = cfg, None

    def validate(self):
        self.cfg.validate()

    def build_engine(self):
        import chatlearn_b200
        from chatlearn_b200.data.data import read_data_path_list
        from chatlearn_b200.models.rollout_module import RolloutModule
        cfg = self.cfg
        chatlearn_b200.init(cfg)
        ra, m = cfg.runtime_args, cfg.models
        policy = RolloutModule("policy")
        reference = PolicyTrainer("reference")
        reward = RewardModel("reward")
        trainer = PolicyTrainer("policy_trainer")
        critic = ValueTrainer("value_trainer") if m.value_trainer is not None else None
        engine = ThreeModelRLHFEngine(policy, reference, reward, trainer, critic)
        engine.set_dataset(read_data_path_list([p.strip() for p in ra.data_path.split(",")]))
        engine.evaluator = None
        engine.set_replay_sample_manager(RlhfAdvantage(
            kl_coef=float(getattr(ra, "init_kl_coef", getattr(m.policy_trainer, "kl_penalty_coef", 0.05)) or 0.0),
            gamma=float(getattr(ra, "gamma", 1.0)), lam=float(getattr(ra, "lam", 0.95)),
            num_inference_per_prompt=int(ra.num_inference_per_prompt)))
        self.engine = engine
        return engine

    def run(self):
        if self.engine is None:
            self.build_engine()
        self.engine.learn()
        return self.engine
