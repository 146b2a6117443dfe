from inferencehackathon_b200.serve.schemas import *  # noqa: F401,F403
