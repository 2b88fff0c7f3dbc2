"""Local scorers: rule-based text rewards, synthetic rewards for random-weight runs, model-based image/video scorers."""
