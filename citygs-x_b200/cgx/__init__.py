"""Host-side mirror of the reference's distributed-render orchestration for the rasterizer hot path:
tile-row workload division (`workload_division`), the Gaussian all-to-all (`exchange`), the dead-but-named
distribution config (`distribution_config`), synthetic scenes (`synthetic`) and a step runner (`runtime`)."""
