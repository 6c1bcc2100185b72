"""Terminal agents that drive a deliverance_b200 server through tool calls."""
