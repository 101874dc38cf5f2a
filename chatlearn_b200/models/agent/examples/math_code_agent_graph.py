"""Math agent with a Python interpreter tool
(chatlearn/models/agent/examples/math_code_agent_graph.py:34-169; the reference runs the
code through agentscope, here it is a child interpreter with a time limit)."""
import subprocess
import sys
import tempfile

from chatlearn_b200.models.agent.agent_module import register
from .tool_agent import ToolLoopAgentGraph, _cfg


def run_python(code: str, timeout: float = 5.0) -> str:
    with tempfile.TemporaryDirectory() as tmp:
        try:
            p = subprocess.run([sys.executable, "-I", "-c", code], capture_output=True, text=True, timeout=timeout,
                               cwd=tmp, env={"PATH": "/usr/bin:/bin"})
            rc, out, err = p.returncode, p.stdout, p.stderr
        except subprocess.TimeoutExpired:
            rc, out, err = -1, "", f"TimeoutError: the code ran longer than {timeout} s"
    return f"<returncode>{rc}</returncode><stdout>{out[-4000:]}</stdout><stderr>{err[-2000:]}</stderr>"


@register("mathcode_agent")
class MathCodeAgentGraph(ToolLoopAgentGraph):
    def tools(self):
        limit = float(_cfg(self.cfg, "code_timeout", 5.0))

        def execute_python(code: str):
            """execute python code and return execute result
            Return the result in the following format:
            <returncode>0</returncode><stdout>the print result in code</stdout><stderr>error message</stderr>

            Args:
                code (str): python code string, must include print to get result
            """
            return run_python(code, limit)

        return [execute_python]
