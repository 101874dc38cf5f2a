from . import geo3k_agent_graph, math_code_agent_graph, math_eval_agent_graph  # noqa: F401
