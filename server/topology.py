from inferencehackathon_b200.serve.topology import *  # noqa: F401,F403
