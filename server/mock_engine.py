from inferencehackathon_b200.serve.mock_engine import *  # noqa: F401,F403
