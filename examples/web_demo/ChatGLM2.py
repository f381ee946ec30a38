#!/usr/bin/env python
"""ChatGLM2 chat demo: web_demo.py with the chatglm2 prompt format, end-of-turn tokens and history depth (prompts.FAMILIES).
Same flags as the reference's examples/web_demo/ChatGLM2.py: -m model dir, -t tokenizer dir, -d dtype, --kv_cache_dtype."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from web_demo import main  # noqa: E402

if __name__ == "__main__":
    main("chatglm2")
