"""Agent graphs, tool parsing and the lock-step trajectory driver (CPU, no engine)."""
import json

from chatlearn_b200.data.tokenizer import ByteTokenizer
from chatlearn_b200.models.agent.base_agent_graph import END, StateGraph
from chatlearn_b200.models.agent.chat_model import ChatModel, HumanMessage, LLMResponse
from chatlearn_b200.models.agent.examples.math_code_agent_graph import MathCodeAgentGraph, run_python
from chatlearn_b200.models.agent.examples.math_eval_agent_graph import MathEvalAgentGraph
from chatlearn_b200.models.agent.rollout_manager import balance_by_tokens
from chatlearn_b200.models.agent.tool_parser import HermesToolParser, ToolParser

TOK = ByteTokenizer(512)


def enc(s):
    return TOK.encode(s)


def test_hermes_parser():
    p = ToolParser.get_tool_parser("hermes", TOK)
    assert isinstance(p, HermesToolParser)
    txt = 'think <tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call> then <tool_call>broken</tool_call> end'
    content, calls = p.extract_tool_calls(enc(txt))
    assert [c.name for c in calls] == ["f"] and json.loads(calls[0].arguments) == {"x": 1}
    assert "tool_call" not in content and content.startswith("think")
    assert p.extract_tool_calls(enc("no tools here")) == ("no tools here", [])


def test_state_graph_routes_and_terminates():
    g = StateGraph()
    g.add_node("a", lambda s, c: {"n": s.get("n", 0) + 1})
    g.add_node("b", lambda s, c: {"n": s["n"] * 10})
    g.set_entry_point("a")
    g.add_conditional_edges("a", lambda s: "again" if s["n"] < 3 else "out", {"again": "a", "out": "b"})
    g.add_edge("b", END)
    assert g.compile().invoke({"messages": []})["n"] == 30


def test_python_tool_runs_in_a_child_with_a_time_limit():
    assert "<returncode>0</returncode><stdout>42\n</stdout>" in run_python("print(6*7)")
    assert "TimeoutError" in run_python("while True: pass", timeout=0.5)


def test_code_agent_two_turns_tokens_and_mask():
    graph = MathCodeAgentGraph("mathcode_agent", cfg={"max_ai_message_turn": 3}, tokenizer=TOK)
    turns = [enc('<tool_call>{"name": "execute_python", "arguments": {"code": "print(6*7)"}}</tool_call>'),
             enc("The answer is 42")]
    seen = []

    def llm(req):
        seen.append(list(req.token_ids))
        return LLMResponse(turns[len(seen) - 1], [-0.5] * len(turns[len(seen) - 1]), "stop")

    gen = graph.run(messages=[{"role": "user", "content": "6*7?"}], sampling_params={}, ground_truth="42")
    try:
        req = next(gen)
        while True:
            req = gen.send(llm(req))
    except StopIteration as e:
        out = e.value
    assert len(seen) == 2 and out.num_turns == 4          # user, ai, tool, ai
    # the second request continues the first trajectory: prompt + turn 1 + tool answer tokens
    assert seen[1][:len(seen[0]) + len(turns[0])] == seen[0] + turns[0]
    assert out.prompt_ids == seen[0]
    assert out.all_token_ids == seen[1] + turns[1]
    n0, n1, n2 = len(seen[0]), len(turns[0]), len(turns[1])
    tool_tokens = len(seen[1]) - n0 - n1
    assert out.loss_mask == [0] * n0 + [1] * n1 + [0] * tool_tokens + [1] * n2
    assert "<stdout>42" in out.str_output and out.str_output.endswith("The answer is 42")
    assert len(out.response_logprobs) == n1 + tool_tokens + n2


def test_turn_limit_and_eval_tool():
    graph = MathEvalAgentGraph("matheval_agent", cfg={"max_ai_message_turn": 2}, tokenizer=TOK)
    call = enc('<tool_call>{"name": "mathlighteval_reward", "arguments": {"answer": "7"}}</tool_call>')
    n = [0]

    def llm(req):
        n[0] += 1
        if n[0] == 2:
            assert "The answer is wrong." in TOK.decode(req.token_ids)
        return LLMResponse(call, None, "stop")

    state_out = None
    gen = graph.run(messages=[HumanMessage("q")], sampling_params={}, ground_truth="8")
    try:
        req = next(gen)
        while True:
            req = gen.send(llm(req))
    except StopIteration as e:
        state_out = e.value
    assert n[0] == 2 and state_out.loss_mask.count(1) == 2 * len(call)   # stopped by the turn limit


def test_chat_model_rejects_bad_tool_arguments():
    cm = ChatModel("m", TOK)
    pre = cm.preprocess([HumanMessage("hi")])
    msg = cm.postprocess(LLMResponse(enc('<tool_call>{"name": "f", "arguments": [1, 2]}</tool_call>')), pre)
    assert not msg.tool_calls and msg.invalid_tool_calls[0]["name"] == "f"


def test_token_balance_groups_have_even_load():
    data = [{"all_token_length": n, "id": i} for i, n in enumerate([100, 90, 80, 70, 10, 20, 30, 40])]
    out = balance_by_tokens(data, 2, 4)
    assert sorted(d["id"] for d in out) == list(range(8))
    a, b = sum(d["all_token_length"] for d in out[:4]), sum(d["all_token_length"] for d in out[4:])
    assert abs(a - b) <= 20


def test_continuous_scheduling_lets_a_trajectory_take_its_next_turn_while_others_decode():
    """Two-turn trajectories with different turn lengths on a real (tiny, CPU) engine: with the open session a
    short trajectory's second turn joins the batch while the long one is still in its first; both schedules
    give the same tokens (greedy sampling)."""
    import torch
    from chatlearn_b200.configs.policy_config import PolicyConfig
    from chatlearn_b200.models.agent.agent_module import AgentModule
    from chatlearn_b200.models.agent.base_agent_graph import AgentGraphOutput, BaseAgentGraph
    from chatlearn_b200.models.agent.chat_model import LLMRequest
    from chatlearn_b200.models.nn import PRESETS, CausalLM
    from chatlearn_b200.rollout import RolloutEngine

    class TwoTurns(BaseAgentGraph):
        def run(self, sampling_params, prompt_ids=None, first=4, **query):
            a = yield LLMRequest(list(prompt_ids), {"max_new_tokens": first}, None)
            b = yield LLMRequest(list(prompt_ids) + list(a.output_ids) + [7], {"max_new_tokens": 3}, None)
            ids = list(prompt_ids) + list(a.output_ids) + [7] + list(b.output_ids)
            return AgentGraphOutput(str_output="", prompt_ids=list(prompt_ids), all_token_ids=ids,
                                    loss_mask=[0] * len(prompt_ids) + [1] * (len(ids) - len(prompt_ids)), num_turns=2)

    arch = PRESETS["tiny_qwen3"]()
    model = CausalLM(arch, dtype=torch.float32).init_weights(2)
    g = torch.Generator().manual_seed(3)
    data = [{"agent_name": "two", "prompt_ids": torch.randint(0, arch.vocab_size - 1, (n,), generator=g).tolist(),
             "first": f} for n, f in ((12, 16), (9, 2), (15, 5))]
    results = {}
    for mode in ("continuous", "lockstep"):
        mod = AgentModule.__new__(AgentModule)
        mod._module_args = PolicyConfig(temperature=0.0, max_response_tokens_length=16, seq_length=128,
                                        agent_scheduling=mode)
        mod.module_args.ignore_eos = True
        mod.engine = RolloutEngine(model, block_size=8, num_blocks=128, max_num_seqs=16, max_model_len=128)
        mod.tp_group = None
        mod.agent_factory = {"two": TwoTurns("two", tokenizer=TOK)}
        outs = mod.run_trajectories(data)
        results[mode] = [o.all_token_ids for o in outs]
        if mode == "continuous":
            st = mod.agent_stats
            assert st["requests"] == 6 and st["joined_running_batch"] >= 2
            # lock-step would need 16 + 3 steps after the prefills; here the second turns overlap the long first turn
            assert st["engine_steps"] <= 16 + 3 + 4
    assert results["continuous"] == results["lockstep"]
    assert [len(t) for t in results["continuous"]] == [12 + 16 + 1 + 3, 9 + 2 + 1 + 3, 15 + 5 + 1 + 3]
