// Stand-in for <glog/logging.h>: the host code is written against the glog macro
// surface the reference uses (LOG(severity), CHECK*, kuiper/include/base/base.h:4),
// and glog itself is not a dependency of this build.
#pragma once
#include "base/log.h"
