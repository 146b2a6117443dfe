from inferencehackathon_b200.serve.backends import *  # noqa: F401,F403
from inferencehackathon_b200.serve.backends import _vllm_healthy  # noqa: F401
