"""Agent layer: tool-using agents that drive an inference engine over several turns and hand trajectories to the trainer."""
