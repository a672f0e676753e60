// Stand-in for <string.h> when a fused chain is compiled at run time: the run-time compiler has the
// declarations built in and no host headers.
#pragma once
