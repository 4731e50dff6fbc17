"""Agent-style workflows: objects with ``async run(data, **extra) -> reward`` that speak the OpenAI
chat-completions protocol. They run through :class:`areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow`
(inline with an engine-bound client, or against the proxy server's ``base_url``)."""

from .math_agent import CALCULATOR_TOOLS, MathAgent, MathToolAgent, MultiTurnMathAgent, math_reward_fn
from .search_agent import HttpSearch, LocalCorpus, ReActSearchAgent, qa_reward
from .service_desk_agent import ServiceDeskAgent, make_desk_tasks
from .terminal_agent import TerminalAgent

__all__ = ["CALCULATOR_TOOLS", "MathAgent", "MathToolAgent", "MultiTurnMathAgent", "math_reward_fn",
           "HttpSearch", "LocalCorpus", "ReActSearchAgent", "qa_reward", "TerminalAgent", "ServiceDeskAgent",
           "make_desk_tasks"]
