from .env import DistEnv
