"""b200fw: a Blackwell (sm_100a) native train / RL / inference framework."""
__version__ = "0.1.0"
