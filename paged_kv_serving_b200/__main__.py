from paged_kv_serving_b200.cli import main

raise SystemExit(main())
