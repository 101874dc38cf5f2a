"""Multi-turn, tool-using rollouts (agent tasks)."""
from .base_agent_graph import AgentGraphOutput, BaseAgentGraph, StateGraph, END  # noqa: F401
from .chat_model import AIMessage, ChatModel, HumanMessage, LLMRequest, LLMResponse, SystemMessage, ToolMessage  # noqa: F401
from .tool_parser import FunctionCall, HermesToolParser, ToolParser  # noqa: F401
