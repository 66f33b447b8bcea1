"""Analysis of sweep results (``results``) and operator wall-clock profiles (``wall_clock``), the roles of zoology/analysis/*."""
